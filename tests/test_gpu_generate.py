"""Generation through the entry points: greedy and temperature sampling against the
plain implementation, stop tokens, batches, and the command line."""
import os
import subprocess
import sys

import pytest
import torch

import plain_mistral as P
import braidinfer_b200 as lib
from braidinfer_b200.sampling import SamplingParams, uniform
from gpu_util import Oracle
from tiny import make_folder, random_prompts

pytestmark = pytest.mark.gpu


def plain_generate(orc, prompt, n, choose):
    toks, out = list(prompt), []
    for step in range(n):
        t = choose(orc.logits(toks)[-1], step, toks)
        out.append(t)
        toks.append(t)
    return out


@pytest.mark.parametrize("name, lengths, steps", [("A", [5, 9, 2], 6), ("B", [1, 12, 7, 20], 10)])
def test_greedy_generation_float32_equals_plain(name, lengths, steps, tmp_path):
    folder = make_folder(tmp_path, name)
    orc = Oracle(folder)
    prompts = random_prompts(orc.cfg.vocab_size, lengths, seed=21)
    m = lib.load(folder, dtype="float32", max_seq_len=128, max_batch=4, verbose=False)
    outs = m.generate(prompts, SamplingParams.greedy(), stop_tokens=(), max_new_tokens=steps)
    for p, o in zip(prompts, outs):
        assert o.finish_reason == "length" and o.prompt_tokens == len(p)
        assert o.tokens == plain_generate(orc, p, steps, lambda lg, s, h: P.argmax_lowest(lg))
    one = m.generate_from_ids(prompts[1], max_tokens=4)             # one prompt in, token ids out
    assert one == outs[1].tokens[:4]
    assert m.engine.cache.slots.available == 4 and m.engine.cache.pages_in_use() == [0]


def test_greedy_generation_bfloat16_follows_the_plain_logits(tmp_path):
    folder = make_folder(tmp_path, "A")
    orc = Oracle(folder)
    prompts = random_prompts(orc.cfg.vocab_size, [5, 9, 2], seed=21)
    m = lib.load(folder, dtype="bfloat16", max_seq_len=128, max_batch=4, verbose=False)
    outs = m.generate(prompts, SamplingParams.greedy(), stop_tokens=(), max_new_tokens=6)
    for p, o in zip(prompts, outs):
        toks = list(p)
        for t in o.tokens:                       # each choice is the plain argmax up to bfloat16 rounding
            lg = orc.logits(toks)[-1]
            assert lg[t] >= lg.max() - 3e-2
            toks.append(t)


def test_temperature_sampling_is_seeded_and_matches_the_plain_chain(tmp_path):
    folder = make_folder(tmp_path, "A")
    orc = Oracle(folder)
    prompts = random_prompts(orc.cfg.vocab_size, [5, 9, 2], seed=21)
    m = lib.load(folder, dtype="float32", max_seq_len=128, max_batch=4, verbose=False)
    sp = SamplingParams(temperature=0.8, seed=1)
    a = m.generate(prompts, sp, stop_tokens=(), max_new_tokens=6)
    b = m.generate(prompts, sp, stop_tokens=(), max_new_tokens=6)
    c = m.generate(prompts, SamplingParams(temperature=0.8, seed=2), stop_tokens=(), max_new_tokens=6)
    assert [o.tokens for o in a] == [o.tokens for o in b] != [o.tokens for o in c]
    alone = m.generate([prompts[1]], sp, stop_tokens=(), max_new_tokens=6)      # same draws outside the batch?
    for i, (p, o) in enumerate(zip(prompts, a)):
        toks = list(p)
        for step, t in enumerate(o.tokens):
            u = uniform(1, i, step)
            want = P.sample(orc.logits(toks)[-1], temperature=0.8, top_k=50, u=u)
            if t != want:
                near = {P.sample(orc.logits(toks)[-1], temperature=0.8, top_k=50, u=u + d) for d in (-1e-4, 1e-4)}
                assert t in near
            toks.append(t)
    # a sequence's draws depend on its own index in the request list, not on the batch around it
    assert alone[0].tokens != [] and len(alone[0].tokens) == 6


def test_stop_tokens_and_batches_one_after_another(tmp_path):
    folder = make_folder(tmp_path, "A")
    orc = Oracle(folder)
    prompts = random_prompts(orc.cfg.vocab_size, [4, 6, 3, 8, 5], seed=30)
    m = lib.load(folder, dtype="float32", max_seq_len=64, max_batch=2, verbose=False)    # 5 requests, 2 at a time
    free = m.generate(prompts, SamplingParams.greedy(), stop_tokens=(), max_new_tokens=8)
    assert m.last_stats.batches == 3
    stop = free[0].tokens[3]
    outs = m.generate(prompts, SamplingParams.greedy(), stop_tokens=[stop], max_new_tokens=8)
    for f, o in zip(free, outs):
        if stop in f.tokens:
            assert o.finish_reason == "stop" and o.tokens == f.tokens[:f.tokens.index(stop)]
        else:
            assert o.finish_reason == "length" and o.tokens == f.tokens
    assert outs[0].finish_reason == "stop" and len(outs[0].tokens) <= 3
    # the model's own eos_token_id (2 in this configuration) is the default stop token
    dflt = m.generate(prompts, SamplingParams.greedy(), max_new_tokens=8)
    assert all(2 not in o.tokens for o in dflt)
    assert m.engine.cache.slots.available == 2 and m.engine.cache.pages_in_use() == [0]


def test_command_line(tmp_path):
    folder = make_folder(tmp_path, "A")
    orc = Oracle(folder)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, MODEL=folder, MAX_TOKENS="5", RAW="1", DTYPE="float32")
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "generate"), "7, 200, 31"], env=env,
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr
    want = []
    toks = [7, 200, 31]
    for _ in range(5):
        t = P.argmax_lowest(orc.logits(toks)[-1])
        if t == 2:
            break
        want.append(t)
        toks.append(t)
    assert [int(x) for x in p.stdout.split()] == want
    assert "PPTG pp=" in p.stderr and "tok/s" in p.stderr and "stop tokens: [2]" in p.stderr
    # the folder as first argument instead of MODEL=, and the default prompt
    env.pop("MODEL")
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "generate"), folder], env=env, capture_output=True,
                       text=True, timeout=600)
    assert p.returncode == 0, p.stderr
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "generate")], env=env, capture_output=True, text=True)
    assert p.returncode == 2 and "MODEL" in p.stderr
