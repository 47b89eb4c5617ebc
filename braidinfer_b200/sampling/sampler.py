"""Chooses the next token of every sequence of a batch on the device.

Rows that are plainly greedy go through the argmax kernel; everything else through
the sampling kernel, which applies the reference's chain in its order
(crates/braidinfer-runtime/src/sampling.rs:49-171).  The uniform number of each draw
comes from `rng.uniform(seed, sequence, step)`.
"""
from __future__ import annotations

from collections import Counter
from typing import List, Optional, Sequence

import numpy as np
import torch

from .params import SamplingParams
from .rng import entropy_seed, uniform


class Sampler:
    # The device's error flags are sticky; they are read every this many draws (and by
    # `Engine.check()` whenever the caller wants), not after every draw.
    CHECK_EVERY = 32

    def __init__(self, kernels, device) -> None:
        self.K = kernels
        self.device = device
        self._draws = 0
        self._stages = []            # (pinned int32, device int32, event of the last copy), used in turn
        self._turn = 0
        self._work_buf: Optional[torch.Tensor] = None

    def _stage(self, words: np.ndarray) -> torch.Tensor:
        """Copy a step's option words to the device through pinned memory without blocking the
        host; three buffers in turn, each waiting for its own last copy only."""
        n = int(words.size)
        if len(self._stages) < 3:
            self._stages.append([None, None, None])
        st = self._stages[self._turn % len(self._stages)]
        self._turn += 1
        if st[0] is None or st[0].numel() < n:
            cap = max(1024, 1 << (n - 1).bit_length())
            st[0] = torch.empty(cap, dtype=torch.int32, pin_memory=True)
            st[1] = torch.empty(cap, dtype=torch.int32, device=self.device)
            st[2] = None
        if st[2] is not None:
            st[2].synchronize()
        st[0].numpy()[:n] = words
        st[1][:n].copy_(st[0][:n], non_blocking=True)
        st[2] = torch.cuda.Event()
        st[2].record()
        return st[1]

    def _work(self, rows: int, vocab: int) -> torch.Tensor:
        if self._work_buf is None or self._work_buf.numel() < rows * vocab:
            self._work_buf = torch.empty(rows * vocab, dtype=torch.float32, device=self.device)
        return self._work_buf[:rows * vocab].view(rows, vocab)

    def choose(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               sequence_ids: Sequence[int], steps: Sequence[int], histories=None) -> List[int]:
        """logits [rows, vocab] float32 on the device -> one token id per row (host ints).
        `histories` is a list, or a function returning the list, of what the repetition
        penalty looks at for each row (prompt + generated); it is only asked for when some
        row has a penalty."""
        rows, vocab = logits.shape
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        if all(p.is_plain_greedy for p in params):
            self.K.argmax(logits, out)
            return self._read(out)
        f = np.zeros((5, rows), dtype=np.float32)      # temperature, top_p, min_p, rep_penalty, uniform
        k = np.zeros(rows, dtype=np.int32)
        if callable(histories):
            histories = histories() if any(p.repetition_penalty != 1.0 for p in params) else None
        hist_off, hist_tok, hist_cnt = [0], [], []
        bias_off, bias_tok, bias_val = [0], [], []
        for i, p in enumerate(params):
            f[0, i], f[1, i], f[2, i], f[3, i] = p.temperature, p.top_p, p.min_p, p.repetition_penalty
            f[4, i] = uniform(seeds[i], sequence_ids[i], steps[i])
            k[i] = p.top_k
            if p.repetition_penalty != 1.0 and histories is not None:
                for tok, cnt in Counter(histories[i]).items():
                    hist_tok.append(tok)
                    hist_cnt.append(cnt)
            hist_off.append(len(hist_tok))
            if p.logit_bias:
                for tok, delta in p.logit_bias:
                    bias_tok.append(tok)
                    bias_val.append(delta)
            bias_off.append(len(bias_tok))
        fd = torch.from_numpy(f).to(self.device)
        ints = np.concatenate([k, np.asarray(hist_off, np.int32), np.asarray(bias_off, np.int32),
                               np.asarray(hist_tok, np.int32), np.asarray(hist_cnt, np.int32),
                               np.asarray(bias_tok, np.int32)]).astype(np.int32)
        idev = torch.from_numpy(ints).to(self.device)
        o = 0
        kd = idev[o:o + rows]; o += rows
        ho = idev[o:o + rows + 1]; o += rows + 1
        bo = idev[o:o + rows + 1]; o += rows + 1
        ht = idev[o:o + len(hist_tok)]; o += len(hist_tok)
        hc = idev[o:o + len(hist_cnt)]; o += len(hist_cnt)
        bt = idev[o:o + len(bias_tok)]
        bv = torch.tensor(bias_val, dtype=torch.float32, device=self.device) if bias_val else None
        work = torch.empty((rows, vocab), dtype=torch.float32, device=self.device)
        self.K.sample(logits, work, out, fd[0], fd[4], top_k=kd, top_p=fd[1], min_p=fd[2], rep_penalty=fd[3],
                      hist_off=ho, hist_tok=ht if hist_tok else None, hist_cnt=hc if hist_cnt else None,
                      bias_off=bo, bias_tok=bt if bias_tok else None, bias_val=bv)
        return self._read(out)

    def choose_async(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
                     sequence_ids: Sequence[int], steps: Sequence[int]) -> "PendingTokens":
        """Like `choose` for rows that need no history (no repetition penalty): launches the
        choice and the copy of the tokens to pinned host memory and returns at once.  The
        tokens stay on the device too (`PendingTokens.device`), where the next step can read them."""
        if any(p.repetition_penalty != 1.0 for p in params):
            raise ValueError("choose_async cannot apply a repetition penalty: it needs the tokens on the host")
        rows, vocab = logits.shape
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        if all(p.is_plain_greedy for p in params):
            self.K.argmax(logits, out)
        else:
            f = np.zeros((4, rows), dtype=np.float32)
            k = np.zeros(rows, dtype=np.int32)
            bias_off, bias_tok, bias_val = [0], [], []
            for i, p in enumerate(params):
                f[0, i], f[1, i], f[2, i] = p.temperature, p.top_p, p.min_p
                f[3, i] = uniform(seeds[i], sequence_ids[i], steps[i])
                k[i] = p.top_k
                for tok, delta in (p.logit_bias or ()):
                    bias_tok.append(tok)
                    bias_val.append(delta)
                bias_off.append(len(bias_tok))
            # every option of the step in one pinned buffer and one copy that does not wait
            nb = len(bias_tok)
            words = np.concatenate([f.reshape(-1).view(np.int32), k, np.asarray(bias_off, np.int32),
                                    np.asarray(bias_tok, np.int32), np.asarray(bias_val, np.float32).view(np.int32)])
            dev = self._stage(words)
            fd = dev[:4 * rows].view(torch.float32).view(4, rows)
            o = 4 * rows
            kd = dev[o:o + rows]; o += rows
            bo = dev[o:o + rows + 1]; o += rows + 1
            bt = dev[o:o + nb] if nb else None; o += nb
            bv = dev[o:o + nb].view(torch.float32) if nb else None
            work = self._work(rows, vocab)
            self.K.sample(logits, work, out, fd[0], fd[3], top_k=kd, top_p=fd[1], min_p=fd[2],
                          bias_off=bo, bias_tok=bt, bias_val=bv)
        host = torch.empty(rows, dtype=torch.int32, pin_memory=True)
        host.copy_(out, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return PendingTokens(self, out, host, done)

    def _read(self, out: torch.Tensor) -> List[int]:
        toks = out.tolist()                    # synchronises: the step's results are complete here
        self._draws += 1
        if self._draws % self.CHECK_EVERY == 0:
            self.K.check_device_errors()
        return toks


class PendingTokens:
    """Tokens chosen on the device whose copy to the host is under way."""

    def __init__(self, sampler: Sampler, device: torch.Tensor, host: torch.Tensor, done) -> None:
        self.sampler, self.device, self.host, self.done = sampler, device, host, done

    def read(self) -> List[int]:
        self.done.synchronize()
        s = self.sampler
        s._draws += 1
        if s._draws % s.CHECK_EVERY == 0:
            s.K.check_device_errors()
        return self.host.tolist()
