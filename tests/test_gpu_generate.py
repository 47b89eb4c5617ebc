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
    for i, (p, o) in enumerate(zip(prompts, a)):
        toks = list(p)
        for step, t in enumerate(o.tokens):
            u = uniform(1, i, step)
            want = P.sample(orc.logits(toks)[-1], temperature=0.8, top_k=50, u=u)
            if t != want:
                near = {P.sample(orc.logits(toks)[-1], temperature=0.8, top_k=50, u=u + d) for d in (-1e-4, 1e-4)}
                assert t in near
            toks.append(t)


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


def run_cli(args, **env):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    e = dict(os.environ, RAW="1")
    e.update({k: str(v) for k, v in env.items()})
    return subprocess.run([sys.executable, os.path.join(root, "bin", "generate")] + list(args), env=e,
                          capture_output=True, text=True, timeout=600)


def test_command_line_sampling_options_are_seeded(tmp_path):
    folder = make_folder(tmp_path, "A")
    opts = dict(MODEL=folder, MAX_TOKENS=8, DTYPE="float32", TEMPERATURE="0.9", TOP_K="40", TOP_P="0.95", MIN_P="0.01")
    a = run_cli(["7, 200, 31"], SEED=5, **opts)
    b = run_cli(["7, 200, 31"], SEED=5, **opts)
    c = run_cli(["7, 200, 31"], SEED=6, **opts)
    assert a.returncode == b.returncode == c.returncode == 0, a.stderr + c.stderr
    assert a.stdout == b.stdout != c.stdout and len(a.stdout.split()) <= 8
    # the same options through the Python entry point choose the same tokens
    m = lib.load(folder, dtype="float32", max_batch=1, verbose=False)
    sp = SamplingParams(temperature=0.9, top_k=40, top_p=0.95, min_p=0.01, seed=5)
    assert [int(x) for x in a.stdout.split()] == m.generate([7, 200, 31], sp, None, 8)
    # a repetition penalty takes the loop that reads every token back; greedy with a penalty differs from plain greedy
    g = run_cli(["7, 7, 7, 7"], MODEL=folder, MAX_TOKENS=6, DTYPE="float32")
    r = run_cli(["7, 7, 7, 7"], MODEL=folder, MAX_TOKENS=6, DTYPE="float32", TEMPERATURE="0.0001", TOP_K="1",
                REPETITION_PENALTY="50", SEED=1)
    assert g.returncode == 0 and r.returncode == 0, g.stderr + r.stderr
    rt = [int(x) for x in r.stdout.split()]
    assert len(set(rt)) == len(rt)                            # a penalty of 50 never lets a token come twice
    bad = run_cli(["7"], MODEL=folder, TEMPERATURE="warm")
    assert bad.returncode != 0 and "TEMPERATURE" in bad.stderr


def test_command_line_batch_file_and_max_seq_len(tmp_path):
    folder = make_folder(tmp_path, "A")
    orc = Oracle(folder)
    lines = ["7, 200, 31", "5", "9, 9, 100, 3, 77, 12"]
    bf = tmp_path / "prompts.txt"
    bf.write_text("\n".join(lines) + "\n\n")
    p = run_cli([], MODEL=folder, MAX_TOKENS=5, DTYPE="float32", BATCH_FILE=str(bf), MAX_SEQ_LEN=64)
    assert p.returncode == 0, p.stderr
    got = [[int(x) for x in l.split()] for l in p.stdout.strip("\n").split("\n")]
    assert len(got) == 3
    for line, g in zip(lines, got):
        toks, want = [int(x) for x in line.replace(",", " ").split()], []
        for _ in range(5):
            t = P.argmax_lowest(orc.logits(toks)[-1])
            if t == 2:
                break
            want.append(t)
            toks.append(t)
        assert g == want
    assert "max_seq_len: 64" in p.stderr                      # the cache holds 64 positions a sequence
    # a request that cannot fit the cache MAX_SEQ_LEN asked for is refused in words
    p = run_cli([", ".join(["3"] * 60)], MODEL=folder, MAX_TOKENS=10, DTYPE="float32", MAX_SEQ_LEN=64)
    assert p.returncode == 2 and "the cache holds 64" in p.stderr
    p = run_cli([", ".join(["3"] * 60)], MODEL=folder, MAX_TOKENS=10, DTYPE="float32", MAX_SEQ_LEN=128)
    assert p.returncode == 0 and "max_seq_len: 128" in p.stderr


def test_command_line_with_a_tokenizer_prepends_bos(tmp_path):
    pytest.importorskip("tokenizers")
    import json
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace
    folder = make_folder(tmp_path, "A")                      # bos_token_id 1, eos_token_id 2
    vocab = {f"w{i}": i for i in range(256)}
    t = Tokenizer(WordLevel(vocab, unk_token="w0"))
    t.pre_tokenizer = Whitespace()
    t.save(os.path.join(folder, "tokenizer.json"))
    orc = Oracle(folder)
    p = run_cli(["w7 w200 w31"], MODEL=folder, MAX_TOKENS=4, DTYPE="float32")
    assert p.returncode == 0, p.stderr
    toks, want = [1, 7, 200, 31], []                          # BOS first
    for _ in range(4):
        tok = P.argmax_lowest(orc.logits(toks)[-1])
        if tok == 2:
            break
        want.append(tok)
        toks.append(tok)
    assert p.stdout.split() == [f"w{i}" for i in want]
    with open(os.path.join(folder, "tokenizer_config.json"), "w") as f:
        json.dump({"add_bos_token": False}, f)
    q = run_cli(["w7 w200 w31"], MODEL=folder, MAX_TOKENS=4, DTYPE="float32")
    first = P.argmax_lowest(orc.logits([7, 200, 31])[-1])
    assert q.returncode == 0 and (q.stdout.split()[:1] == [f"w{first}"] or first == 2)


def fnv_of_float32(row: torch.Tensor) -> int:
    """The hash of crates/braidinfer-runtime/src/generate.rs:385-389, element by element."""
    h = 0xcbf29ce484222325
    for bits in row.contiguous().view(torch.int32).tolist():
        h ^= bits & 0xFFFFFFFF
        h = (h * 0x100000001b3) & 0xFFFFFFFFFFFFFFFF
    return h


def test_logit_trace_file_names_every_step(tmp_path, monkeypatch):
    """BRAIDINFER_LOGIT_TRACE: the hashes are those of the logits a replay of the same tokens gives (so equal runs
    write equal files), the kernel's hash is the reference's, and with the variable set the tokens stay the same."""
    folder = make_folder(tmp_path, "A")
    m = lib.load(folder, dtype="bfloat16", max_seq_len=128, max_batch=2, verbose=False)
    prompts = random_prompts(m.config.vocab_size, [7, 3], seed=8)
    plain = m.generate(prompts, SamplingParams.greedy(), stop_tokens=(), max_new_tokens=4)
    path = tmp_path / "logits.txt"
    monkeypatch.setenv("BRAIDINFER_LOGIT_TRACE", str(path))
    traced = m.generate(prompts, SamplingParams.greedy(), stop_tokens=(), max_new_tokens=4)
    first = path.read_text()
    m.generate(prompts, SamplingParams.greedy(), stop_tokens=(), max_new_tokens=4)
    monkeypatch.delenv("BRAIDINFER_LOGIT_TRACE")
    assert [o.tokens for o in traced] == [o.tokens for o in plain]
    assert path.read_text() == first + first                        # appended, and the same bits again
    lines = first.splitlines()
    assert len(lines) == 8
    # the same tokens through the step function: prompt, then one token each
    slots = [m.open(), m.open()]
    logits = [m.step(list(zip(slots, prompts)), want="last")]
    for t in range(3):
        logits.append(m.step([(s, [o.tokens[t]]) for s, o in zip(slots, plain)], want="last"))
    for s in slots:
        m.close(s)
    for k in range(4):
        for i in range(2):
            row = logits[k][i].float().cpu()
            assert lines[2 * k + i] == f"step={k} tok={plain[i].tokens[k]} logit_hash={fnv_of_float32(row):016x} seq={i}"
    # the kernel by itself, at a width that is no multiple of its chunk
    g = torch.Generator().manual_seed(3)
    x = torch.randn(3, 4096 + 37, generator=g).cuda()
    assert m.engine.kernels.logit_hash(x) == [fnv_of_float32(r) for r in x.cpu()]
