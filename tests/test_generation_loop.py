"""The generation loop's decisions, on the CPU, with a stand-in engine whose "model"
is a fixed rule: the next token after token t is (t + 1) % vocab."""
import pytest
import torch

from braidinfer_b200.engine.generate import GenerationLoop, plan_batches
from braidinfer_b200.sampling import SamplingParams

VOCAB = 50


class FakeEngine:
    def __init__(self, max_tokens=64 * 4, max_slots=4):
        self.max_tokens, self.max_slots = max_tokens, max_slots
        self.free = list(range(max_slots))
        self.live = {}
        self.calls = []
        self.closed = []

    def open(self):
        s = self.free.pop(0)
        self.live[s] = []
        return s

    def close(self, s):
        assert s in self.live, "slot freed twice"
        del self.live[s]
        self.free.append(s)
        self.closed.append(s)

    def step(self, entries, want="last"):
        assert want == "last"
        self.calls.append([(s, list(t)) for s, t in entries])
        out = torch.full((len(entries), VOCAB), -1.0)
        for i, (s, t) in enumerate(entries):
            self.live[s].extend(t)
            out[i, (t[-1] + 1) % VOCAB] = 1.0
        return out


class ArgmaxSampler:
    def choose(self, logits, params, seeds, ids, steps, hist):
        self.last = (list(ids), list(steps), [list(h) for h in hist()])
        return logits.argmax(-1).tolist()


def test_plan_batches_respects_count_and_capacity():
    assert plan_batches([5, 5, 5], [10, 10, 10], 64 * 8, 2) == [[0, 1], [2]]
    assert plan_batches([60, 60, 60], [10, 10, 10], 256, 8) == [[0, 1], [2]]      # 128 tokens each after rounding
    assert plan_batches([], [], 64, 4) == []
    with pytest.raises(ValueError, match="request 1"):
        plan_batches([5, 100], [5, 100], 128, 4)


def test_prompt_in_one_step_then_one_token_each():
    eng, smp = FakeEngine(), ArgmaxSampler()
    out = GenerationLoop(eng, smp).generate([[3, 4, 5], [10]], max_new_tokens=3)
    assert [o.tokens for o in out] == [[6, 7, 8], [11, 12, 13]]
    assert all(o.finish_reason == "length" for o in out)
    assert eng.calls[0] == [(0, [3, 4, 5]), (1, [10])]                # both prompts in the first step
    assert eng.calls[1] == [(0, [6]), (1, [11])]
    assert len(eng.calls) == 3                                        # no step after the last token
    assert not eng.live and sorted(eng.closed) == [0, 1]


def test_stop_token_is_not_returned_and_frees_the_slot_at_once():
    eng = FakeEngine()
    out = GenerationLoop(eng, ArgmaxSampler()).generate([[1], [20]], max_new_tokens=6, stop_tokens=[4])
    assert out[0].tokens == [2, 3] and out[0].finish_reason == "stop"
    assert out[1].tokens == [21, 22, 23, 24, 25, 26] and out[1].finish_reason == "length"
    assert eng.closed[0] == 0                                          # the shorter one left first
    assert eng.calls[3] == [(1, [23])]                                 # and the batch went on without it
    # a stop token as the very first choice: nothing is emitted
    out = GenerationLoop(FakeEngine(), ArgmaxSampler()).generate([[3]], max_new_tokens=5, stop_tokens=[4])
    assert out[0].tokens == [] and out[0].finish_reason == "stop"


def test_batches_follow_one_another_and_reuse_slots():
    eng = FakeEngine(max_tokens=64 * 2, max_slots=2)
    prompts = [[i] for i in range(5)]
    out = GenerationLoop(eng, ArgmaxSampler(), max_batch=8).generate(prompts, max_new_tokens=[1, 2, 3, 1, 2])
    assert [o.tokens for o in out] == [[1], [2, 3], [3, 4, 5], [4], [5, 6]]
    assert [len(c) for c in eng.calls] == [2, 1, 2, 1, 1, 1, 1]
    assert not eng.live and len(eng.closed) == 5 and set(eng.closed) == {0, 1}


def test_per_sequence_step_counters_and_histories_reach_the_sampler():
    eng, smp = FakeEngine(), ArgmaxSampler()
    GenerationLoop(eng, smp).generate([[7, 8], [30]], max_new_tokens=[3, 1])
    ids, steps, hist = smp.last
    assert ids == [0] and steps == [2] and hist == [[7, 8, 9, 10]]


def test_edge_cases():
    loop = GenerationLoop(FakeEngine(), ArgmaxSampler())
    with pytest.raises(ValueError, match="empty"):
        loop.generate([[]])
    out = loop.generate([[5]], max_new_tokens=0)
    assert out[0].tokens == [] and out[0].finish_reason == "length"
    with pytest.raises(ValueError):
        loop.generate([[5], [6]], params=[SamplingParams.greedy()])

    class Boom(FakeEngine):
        def step(self, entries, want="last"):
            if len(self.calls) == 1:
                raise RuntimeError("boom")
            return super().step(entries, want)

    eng = Boom()
    with pytest.raises(RuntimeError):
        GenerationLoop(eng, ArgmaxSampler()).generate([[1], [2]], max_new_tokens=4)
    assert not eng.live                                               # nothing stays held after an error


class DeviceTokenEngine(FakeEngine):
    """A stand-in whose step can take its tokens from a tensor the sampler left behind."""

    def step(self, entries, want="last", device_tokens=None):
        if device_tokens is not None:
            tensor, rows = device_tokens
            entries = [(s, [int(tensor[r])]) for (s, _), r in zip(entries, rows)]
        return super().step(entries, want)


class AsyncArgmaxSampler(ArgmaxSampler):
    class Pending:
        def __init__(self, toks):
            self.device = torch.tensor(toks, dtype=torch.int32)
            self._toks = toks

        def read(self):
            return list(self._toks)

    def choose_async(self, logits, params, seeds, ids, steps):
        self.async_calls = getattr(self, "async_calls", 0) + 1
        return self.Pending(logits.argmax(-1).tolist())


def test_pipelined_loop_makes_the_same_decisions():
    prompts = [[1], [20], [7, 8]]
    kw = dict(max_new_tokens=[6, 6, 2], stop_tokens=[4])
    want = GenerationLoop(FakeEngine(), ArgmaxSampler()).generate(prompts, **kw)
    eng, smp = DeviceTokenEngine(), AsyncArgmaxSampler()
    got = GenerationLoop(eng, smp).generate(prompts, **kw)
    assert smp.async_calls > 0
    assert [(o.tokens, o.finish_reason) for o in got] == [(o.tokens, o.finish_reason) for o in want]
    assert got[0].tokens == [2, 3] and got[0].finish_reason == "stop"
    assert got[2].tokens == [9, 10] and got[2].finish_reason == "length"
    assert not eng.live and sorted(eng.closed) == [0, 1, 2]
    # the sequence that ends by length is not run past its last token; the one that meets
    # a stop token has run one step too many, whose result is dropped
    fed = {s: [t for call in eng.calls for (slot, toks) in call for t in toks if slot == s] for s in (0, 1, 2)}
    assert fed[2] == [7, 8, 9] and fed[0] == [1, 2, 3, 4] and fed[1] == [20, 21, 22, 23, 24, 25]
    # a repetition penalty needs the tokens on the host: the plain loop runs instead
    from braidinfer_b200.sampling import SamplingParams
    smp2 = AsyncArgmaxSampler()
    GenerationLoop(DeviceTokenEngine(), smp2).generate([[1]], params=SamplingParams(temperature=0.0, repetition_penalty=1.2),
                                                       max_new_tokens=3)
    assert getattr(smp2, "async_calls", 0) == 0


def test_where_a_product_is_spread_along_k():
    """`stream_k_pays` at the points it was measured on (148 SMs, 7B layer sizes): partial sums
    wherever whole tiles would leave SMs idle and the sums are small beside the weights, whole tiles
    where they fill the SMs or the tokens are many."""
    from braidinfer_b200.parts.linear import stream_k_pays
    pays = lambda rows, shape: stream_k_pays(rows, shape[0], shape[1], 148)
    qkv, o, gate_up, down, head = (6144, 4096), (4096, 4096), (2 * 14336, 4096), (4096, 14336), (32768, 4096)
    for rows in (1, 8, 32, 64, 128, 160, 256):
        assert pays(rows, qkv) and pays(rows, o) and pays(rows, down)
    assert pays(8, gate_up) and pays(32, gate_up) and pays(48, gate_up)              # 224 tiles: 76 % full
    assert not any(pays(r, gate_up) for r in (64, 128, 160, 256, 512))
    assert not any(pays(r, head) for r in (1, 8, 64, 512))                           # 256 tiles: 86 % full
    assert not pays(384, qkv) and not pays(384, o) and pays(384, down)               # the sums outweigh k = 4096
    assert not pays(512, o) and pays(512, down) and not pays(512, qkv)
    assert not any(pays(768, s) for s in (qkv, o, down))
    assert not pays(769, o) and not pays(2048, down)


def test_logit_trace_lines(tmp_path, monkeypatch):
    """BRAIDINFER_LOGIT_TRACE: a line per chosen token, counted per request from 0, with the hash the engine
    gives for the logits the token was chosen from; the loop then runs unpipelined, with the same results."""
    class HashingEngine(DeviceTokenEngine):
        def logit_hash(self, logits):
            return [int(row.argmax()) * 0x100000001 for row in logits]

    path = tmp_path / "trace.txt"
    monkeypatch.setenv("BRAIDINFER_LOGIT_TRACE", str(path))
    eng = HashingEngine()
    out = GenerationLoop(eng, AsyncArgmaxSampler()).generate([[3, 4], [20]], max_new_tokens=[3, 2], stop_tokens=[7])
    assert [o.tokens for o in out] == [[5, 6], [21, 22]] and out[0].finish_reason == "stop"
    lines = path.read_text().splitlines()
    assert lines == [f"step=0 tok=5 logit_hash={5 * 0x100000001:016x} seq=0", f"step=0 tok=21 logit_hash={21 * 0x100000001:016x} seq=1",
                     f"step=1 tok=6 logit_hash={6 * 0x100000001:016x} seq=0", f"step=1 tok=22 logit_hash={22 * 0x100000001:016x} seq=1",
                     f"step=2 tok=7 logit_hash={7 * 0x100000001:016x} seq=0"]
    monkeypatch.delenv("BRAIDINFER_LOGIT_TRACE")
    GenerationLoop(HashingEngine(), AsyncArgmaxSampler()).generate([[3]], max_new_tokens=1)
    assert len(path.read_text().splitlines()) == 5            # no variable, no lines
