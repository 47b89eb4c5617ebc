"""Long decoding and the first tokens of a sequence, against the plain implementation,
with peaked attention so that one wrong key shows."""
import pytest
import torch

from gpu_util import TOL, Oracle, engine, max_err, sharpen
from tiny import make_folder, random_prompts

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(name, dtype, tmp_path):
    folder = sharpen(make_folder(tmp_path, name), 6.0)
    orc = Oracle(folder)
    toks = random_prompts(orc.cfg.vocab_size, [330], seed=4)[0]
    want = orc.logits(toks)
    eng = engine(folder, dtype, max_tokens=64 * 6)
    s = eng.open()
    got = [eng.step([(s, toks[:10])], want="all")]
    for t in toks[10:]:
        got.append(eng.step([(s, [t])], want="last"))
    eng.check()
    assert max_err(torch.cat(got), want) < TOL[dtype]


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(name, dtype, tmp_path):
    folder = make_folder(tmp_path, name)
    orc = Oracle(folder)
    toks = random_prompts(orc.cfg.vocab_size, [6], seed=8)[0]
    want = orc.logits(toks)
    eng = engine(folder, dtype)
    for first in (1, 2, 3):                     # a prompt of one, two, three tokens, then one by one
        s = eng.open()
        got = [eng.step([(s, toks[:first])], want="all")]
        for t in toks[first:]:
            got.append(eng.step([(s, [t])], want="last"))
        eng.close(s)
        assert max_err(torch.cat(got), want) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_in_chunks_equals_prompt_whole(dtype, tmp_path):
    folder = sharpen(make_folder(tmp_path, "B"), 6.0)
    orc = Oracle(folder)
    toks = random_prompts(orc.cfg.vocab_size, [200], seed=6)[0]
    eng = engine(folder, dtype)
    s = eng.open()
    got = []
    for lo, hi in [(0, 63), (63, 64), (64, 130), (130, 200)]:
        got.append(eng.step([(s, toks[lo:hi])], want="all"))
    assert max_err(torch.cat(got), orc.logits(toks)) < TOL[dtype]
