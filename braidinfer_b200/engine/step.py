"""The step function: run the tokens that a batch of sequences brings, from the
cache, and return logits at the wanted places.

A step packs its sequences one after another into rows ([sum of lengths, width]);
each row knows its sequence and its position (cache length + offset).  Prompts of
unequal lengths go in one step, later steps bring one token each; a prompt may also
be cut into chunks, because attention always reads keys and values from the cache,
where the step's own tokens were just written.  Rows added as padding belong to no
sequence: they write nothing to the cache and nobody reads them.

The reference has one sequence per model and two entry points, prefill(tokens) and
decode_step(token, position), both returning the last token's logits
(crates/braidinfer-runtime/src/model/state.rs:39-50, model/mod.rs:279-286).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch


@dataclass
class StepContext:
    """Device-side description of one step, read by the kernels."""
    rows: int                         # rows including padding
    n_tokens: int
    n_seqs: int
    token_ids: torch.Tensor           # [rows] int32
    positions: torch.Tensor           # [rows] int32
    token_seq: torch.Tensor           # [rows] int32, sequence index in this step or -1 (padding)
    q_start: torch.Tensor             # [n_seqs] first row of each sequence
    q_len: torch.Tensor               # [n_seqs] rows of each sequence
    kv_before: torch.Tensor           # [n_seqs] cache length before the step
    slot_ids: torch.Tensor            # [n_seqs] slot of each sequence (state area index)
    page_tables: List[torch.Tensor]   # per cache group [n_seqs, blocks] int32
    want_rows: Optional[torch.Tensor]  # [n_want] rows whose logits are wanted
    n_want: int
    max_q_len: int
    max_kv_len: int
    all_decode: bool                  # every sequence brings exactly one token
    # host copies, for parts written in Python (tests' toy parts) and for launch shaping
    host_q_len: Tuple[int, ...] = ()
    host_kv_before: Tuple[int, ...] = ()
    host_slots: Tuple[int, ...] = ()
    # Deferred sums.  In a step of a few tokens a product may leave its partial sums in the
    # GEMM workspace and hand the adding-up to the part that reads the result next, which
    # fuses it with its own work (the next norm, the rotary encoding).  `deferred` maps the
    # tensor that is still to be completed (by its data pointer) to (handle, kind): kind
    # "residual" means tensor += sum, "store" means tensor = sum.  A part that does not
    # know about this calls `resolve(tensor)` first, or is handed a resolved tensor by the
    # block.  At most one sum is deferred at a time.
    deferred: dict = field(default_factory=dict)
    # Row scales.  In a step of few tokens a norm may leave its own scale (rsqrt(mean square + eps), one
    # number a row) to the product that reads its output, if the block says that this reader takes row
    # scales: the norm's output then holds the rows times the norm's weights only, and `row_scales` maps
    # it (by data pointer) to the scale (csrc.api.RowScale).  The reader takes it with `take_row_scale`
    # and owes it to its results; a scale that nobody took by the end of the block is an error.
    row_scales: dict = field(default_factory=dict)
    kernels: object = None

    def defer(self, tensor: torch.Tensor, handle, kind: str) -> None:
        self.deferred[tensor.data_ptr()] = (handle, kind)

    def take_deferred(self, tensor: torch.Tensor):
        """(handle, kind) if `tensor` is waiting for a deferred sum (which the caller now
        owns and must add), else None."""
        return self.deferred.pop(tensor.data_ptr(), None)

    def set_row_scale(self, tensor: torch.Tensor, scale) -> None:
        self.row_scales[tensor.data_ptr()] = scale

    def take_row_scale(self, tensor: torch.Tensor):
        """The row scale that `tensor` still wants applied to whatever is computed from it (the caller
        now owes it), or None."""
        return self.row_scales.pop(tensor.data_ptr(), None)

    def resolve(self, tensor: torch.Tensor) -> torch.Tensor:
        """Complete `tensor` now with the plain reduce kernel, if a sum is deferred on it."""
        d = self.deferred.pop(tensor.data_ptr(), None)
        if d is not None:
            handle, kind = d
            if self.kernels is None:
                from ..csrc.api import get_kernels
                self.kernels = get_kernels()
            if kind == "residual":
                self.kernels.streamk_reduce(handle, tensor, residual=tensor)
            else:
                self.kernels.streamk_reduce(handle, tensor)
        return tensor

    def drop_deferred(self) -> None:
        """Forget sums nobody will read (the step wants no logits)."""
        for handle, _ in self.deferred.values():
            if self.kernels is not None and self.kernels.pending_partial is handle:
                self.kernels.pending_partial = None
        self.deferred.clear()
        self.row_scales.clear()


class _Shaped:
    def __init__(self, shape):
        self.shape = shape


class _Sized:                              # what `StepPacker._context` needs of a table: its size
    def __init__(self, size):
        self.size = size


class StepPacker:
    """Builds a step's integer tables on the host and moves them to the device in one copy."""

    def __init__(self, device, row_multiple: int = 1) -> None:
        self.device = device
        self.row_multiple = max(1, int(row_multiple))
        self._pinned: Optional[torch.Tensor] = None
        self._dev: Optional[torch.Tensor] = None
        self._copied: Optional[torch.cuda.Event] = None
        self.h2d_bytes_last = 0
        self.generation = 0          # grows when the device buffer moves (captured graphs are stale then)

    def _buffers(self, n: int) -> Tuple[torch.Tensor, torch.Tensor]:
        if self._pinned is None or self._pinned.numel() < n:
            cap = max(1 << 18, 1 << (n - 1).bit_length())
            if self._copied is not None:
                self._copied.synchronize()
            self.generation += 1
            self._pinned = torch.empty(cap, dtype=torch.int32, pin_memory=True)
            self._dev = torch.empty(cap, dtype=torch.int32, device=self.device)
        return self._pinned, self._dev

    def pack(self, slots: Sequence[int], tokens: Sequence[Sequence[int]], kv_before: Sequence[int],
             want: Sequence[Sequence[int]], tables: Sequence[np.ndarray], bucket_tables: bool = False,
             token_source_rows: Optional[Sequence[int]] = None, pad_rows_to: int = 0) -> StepContext:
        """`bucket_tables` widens every page table to a power-of-two number of columns (at
        least 8), so that steps of the same shape lay their tables out identically.
        `pad_rows_to`: at least this many rows (the rows past the step's tokens are padding)."""
        n_seqs = len(slots)
        if bucket_tables and all(len(t) == 1 for t in tokens) and all(len(w) <= 1 for w in want):
            return self._pack_one_token_each(slots, tokens, kv_before, want, tables, token_source_rows)
        if token_source_rows is not None:
            raise ValueError("tokens can be taken from the device only in steps of one token a sequence")
        if bucket_tables:
            wide = []
            for t in tables:
                cols = max(8, 1 << (t.shape[1] - 1).bit_length())
                w = np.full((t.shape[0], cols), -1, dtype=np.int32)
                w[:, :t.shape[1]] = t
                wide.append(w)
            tables = wide
        q_len = [len(t) for t in tokens]
        n_tokens = sum(q_len)
        rows = -(-max(n_tokens, int(pad_rows_to)) // self.row_multiple) * self.row_multiple
        token_ids = np.zeros(rows, dtype=np.int32)
        positions = np.zeros(rows, dtype=np.int32)
        token_seq = np.full(rows, -1, dtype=np.int32)
        q_start = np.zeros(n_seqs, dtype=np.int32)
        want_rows: List[int] = []
        r = 0
        for i, (t, before) in enumerate(zip(tokens, kv_before)):
            n = len(t)
            q_start[i] = r
            token_ids[r:r + n] = t
            positions[r:r + n] = np.arange(before, before + n, dtype=np.int32)
            token_seq[r:r + n] = i
            for w in want[i]:
                if not (0 <= w < n):
                    raise IndexError(f"wanted place {w} is outside the {n} tokens that sequence {i} brings")
                want_rows.append(r + w)
            r += n
        parts = [token_ids, positions, token_seq, q_start, np.asarray(q_len, dtype=np.int32),
                 np.asarray(kv_before, dtype=np.int32), np.asarray(slots, dtype=np.int32),
                 np.asarray(want_rows, dtype=np.int32)] + [t.reshape(-1) for t in tables]
        # every table starts on a 16-byte boundary
        offs, total = [], 0
        for p in parts:
            offs.append(total)
            total += -(-p.size // 4) * 4
        pinned, dev = self._buffers(max(total, 4))
        if self._copied is not None:
            self._copied.synchronize()          # the last copy out of the pinned buffer is done
        pn = pinned.numpy()
        for p, o in zip(parts, offs):
            pn[o:o + p.size] = p
        dev[:total].copy_(pinned[:total], non_blocking=True)
        self._copied = torch.cuda.Event()
        self._copied.record()
        self.h2d_bytes_last = total * 4

        return self._context(dev, parts, offs, tables, rows, n_tokens, n_seqs, q_len, kv_before, slots, want_rows)

    def _pack_one_token_each(self, slots, tokens, kv_before, want, tables, token_source_rows=None) -> StepContext:
        """The same layout as `pack` for the common step of generation (one token a
        sequence, page tables widened to a power-of-two width), written straight into the
        pinned buffer."""
        n = len(slots)
        rows = -(-n // self.row_multiple) * self.row_multiple
        want_rows = [i for i, w in enumerate(want) if w]
        for w in want:
            if w and w[0] != 0:
                raise IndexError(f"wanted place {w[0]} is outside the 1 token that the sequence brings")
        wide = []
        for t in tables:
            cols = max(8, 1 << (t.shape[1] - 1).bit_length())
            wide.append((t, cols))
        sizes = [rows, rows, rows, n, n, n, n, len(want_rows)] + [n * c for _, c in wide] + [n]
        offs, total = [], 0
        for sz in sizes:
            offs.append(total)
            total += -(-sz // 4) * 4
        pinned, dev = self._buffers(max(total, 4))
        if self._copied is not None:
            self._copied.synchronize()
        pn = pinned.numpy()
        ar = np.arange(n, dtype=np.int32)
        pn[offs[0]:offs[0] + rows] = 0
        pn[offs[0]:offs[0] + n] = [t[0] for t in tokens]
        pn[offs[1]:offs[1] + rows] = 0
        pn[offs[1]:offs[1] + n] = kv_before
        pn[offs[2]:offs[2] + rows] = -1
        pn[offs[2]:offs[2] + n] = ar
        pn[offs[3]:offs[3] + n] = ar
        pn[offs[4]:offs[4] + n] = 1
        pn[offs[5]:offs[5] + n] = kv_before
        pn[offs[6]:offs[6] + n] = slots
        pn[offs[7]:offs[7] + len(want_rows)] = want_rows
        shapes = []
        for g, (t, cols) in enumerate(wide):
            v = pn[offs[8 + g]:offs[8 + g] + n * cols].reshape(n, cols)
            v[:, :t.shape[1]] = t
            v[:, t.shape[1]:] = -1
            shapes.append((n, cols))
        src_k = 8 + len(wide)                       # where each row's token lies in the sampler's output
        pn[offs[src_k]:offs[src_k] + n] = token_source_rows if token_source_rows is not None else ar
        dev[:total].copy_(pinned[:total], non_blocking=True)
        self._copied = torch.cuda.Event()
        self._copied.record()
        self.h2d_bytes_last = total * 4
        self.token_source_view = dev[offs[src_k]:offs[src_k] + n]

        parts = [_Sized(sz) for sz in sizes]
        return self._context(dev, parts, offs, [_Shaped(s) for s in shapes], rows, n, n, [1] * n, kv_before, slots,
                             want_rows)

    def _context(self, dev, parts, offs, tables, rows, n_tokens, n_seqs, q_len, kv_before, slots, want_rows):
        def view(k: int, shape=None) -> torch.Tensor:
            v = dev[offs[k]:offs[k] + parts[k].size]
            return v if shape is None else v.view(shape)

        return StepContext(
            rows=rows, n_tokens=n_tokens, n_seqs=n_seqs,
            token_ids=view(0), positions=view(1), token_seq=view(2), q_start=view(3), q_len=view(4),
            kv_before=view(5), slot_ids=view(6),
            page_tables=[view(8 + g, tables[g].shape) for g in range(len(tables))],
            want_rows=view(7) if want_rows else None, n_want=len(want_rows),
            max_q_len=max(q_len) if q_len else 0,
            max_kv_len=max((b + n for b, n in zip(kv_before, q_len)), default=0),
            all_decode=all(n == 1 for n in q_len),
            host_q_len=tuple(q_len), host_kv_before=tuple(kv_before), host_slots=tuple(slots))
