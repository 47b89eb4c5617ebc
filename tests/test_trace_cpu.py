"""The replay driver's handling of steps, ids and files, with a stand-in engine (CPU)."""
import json

import numpy as np
import pytest
import torch

from braidinfer_b200.engine.trace import replay


class FakeEngine:
    vocab = 7

    def __init__(self):
        self.next_slot, self.live, self.log = 0, {}, []

    def open(self):
        s = self.next_slot
        self.next_slot += 1
        self.live[s] = 0
        return s

    def close(self, s):
        del self.live[s]

    def step(self, entries, want):
        self.log.append(([s for s, _ in entries], want))
        rows = []
        for (s, toks), w in zip(entries, want):
            for i in w:
                rows.append(torch.full((self.vocab,), float(100 * s + self.live[s] + i)))
            self.live[s] += len(toks)
        return torch.stack(rows) if rows else None

    def check(self):
        pass


def test_replay_writes_wanted_logits_in_order_and_reports_each_step(tmp_path):
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": [0, 2]},
                                {"id": "b", "tokens": [4], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": [5], "want": [0]}, {"id": "b", "tokens": [6], "want": [0]}],
         "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": [7], "want": []}], "end": ["a"]},
        {"step": 7, "entries": [{"id": "b", "tokens": [1, 1], "want": [1]}], "end": ["b"]},
    ]
    said = []
    eng = FakeEngine()
    n = replay(eng, [json.dumps(s) for s in steps] + ["", "  "], str(tmp_path), said.append)
    assert n == 4 and said == ["done 0", "done 1", "done 2", "done 7"]
    a0 = np.fromfile(tmp_path / "0.f32", dtype="<f4").reshape(-1, 7)
    assert a0.shape == (2, 7) and a0[0, 0] == 0 and a0[1, 0] == 2
    a1 = np.fromfile(tmp_path / "1.f32", dtype="<f4").reshape(-1, 7)
    assert a1[:, 0].tolist() == [3.0, 101.0]
    assert not (tmp_path / "2.f32").exists()                 # nothing wanted, nothing written
    a7 = np.fromfile(tmp_path / "7.f32", dtype="<f4").reshape(-1, 7)
    assert a7[0, 0] == 201.0                                 # "b" came back as a new request in a new slot
    assert not eng.live


def test_replay_refuses_to_end_an_unknown_request(tmp_path):
    with pytest.raises(KeyError):
        replay(FakeEngine(), [json.dumps({"step": 0, "entries": [], "end": ["zz"]})], str(tmp_path))
