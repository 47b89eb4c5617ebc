"""Trace replay on the GPU: the same requests whole, with their last 32 tokens one by
one, and in batches of unequal lengths whose shorter requests end earlier, one batch
after another so that slots and pages are used again; float32 and bfloat16; every
logit compared with the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from gpu_util import TOL, Oracle, engine, max_err, sharpen
from tiny import CONFIGS, make_folder, random_prompts
from braidinfer_b200.engine.trace import replay

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 9, 2, 70, 33], "B": [1, 12, 7, 20, 75], "C": [3, 140, 64, 65, 17]}


@pytest.fixture(scope="module", params=["A", "B", "C"])
def model(request, tmp_path_factory):
    name = request.param
    folder = sharpen(make_folder(tmp_path_factory.mktemp("m" + name), name), 5.0)
    orc = Oracle(folder)
    prompts = random_prompts(orc.cfg.vocab_size, LENGTHS[name], seed=11)
    return name, folder, orc, prompts


def run_trace(eng, steps, tmp_path):
    out = str(tmp_path)
    said = []
    replay(eng, [json.dumps(s) for s in steps], out, said.append)
    assert said == [f"done {s['step']}" for s in steps]
    got = {}
    for s in steps:
        n_want = sum(len(e["want"]) for e in s["entries"])
        path = os.path.join(out, f"{s['step']}.f32")
        if n_want == 0:
            assert not os.path.exists(path)
            continue
        arr = np.fromfile(path, dtype="<f4").reshape(n_want, eng.vocab_size)
        r = 0
        for e in s["entries"]:
            for w in e["want"]:
                got[(e["id"], e["_start"] + w)] = torch.from_numpy(arr[r].copy())
                r += 1
    return got


def check(got, orc, requests, tol):
    assert got, "nothing was compared"
    worst = 0.0
    for (rid, pos), lg in got.items():
        worst = max(worst, max_err(lg, orc.logits(requests[rid])[pos]))
    assert worst < tol, f"max |logit - plain| = {worst}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_each_request_alone_and_whole(model, dtype, tmp_path):
    name, folder, orc, prompts = model
    eng = engine(folder, dtype, max_tokens=64 * 3)           # room for the longest request only
    requests = {f"r{i}": p for i, p in enumerate(prompts)}
    steps = [{"step": i, "entries": [{"id": rid, "tokens": p, "want": list(range(len(p))), "_start": 0}],
              "end": [rid]} for i, (rid, p) in enumerate(requests.items())]
    check(run_trace(eng, steps, tmp_path), orc, requests, TOL[dtype])
    assert eng.cache.pages_in_use() == [0] * len(eng.cache.groups) and eng.cache.slots.available == eng.max_slots


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_last_32_tokens_one_by_one(model, dtype, tmp_path):
    name, folder, orc, prompts = model
    eng = engine(folder, dtype, max_tokens=64 * 3)
    g = torch.Generator().manual_seed(5)
    requests, steps, k = {}, [], 0
    for i, total in enumerate([33, 70, 100]):                 # prefixes of 1, 38 and 68 tokens
        toks = torch.randint(0, orc.cfg.vocab_size, (total,), generator=g).tolist()
        rid = f"q{i}"
        requests[rid] = toks
        head = total - 32
        steps.append({"step": k, "entries": [{"id": rid, "tokens": toks[:head], "want": [head - 1], "_start": 0}],
                      "end": []})
        k += 1
        for j in range(head, total):
            steps.append({"step": k, "entries": [{"id": rid, "tokens": [toks[j]], "want": [0], "_start": j}],
                          "end": [rid] if j == total - 1 else []})
            k += 1
    check(run_trace(eng, steps, tmp_path), orc, requests, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_one_after_another(model, dtype, tmp_path):
    name, folder, orc, prompts = model
    g = torch.Generator().manual_seed(9)
    # three batches; each request: a prompt and some decoded tokens; the shorter ones end earlier
    plans = [[(5, 6), (9, 2), (2, 9)], [(1, 10), (12, 3), (7, 10), (20, 1)], [(70, 4), (3, 66), (64, 1)]]
    # the cache has room for exactly the largest batch (each request rounded up to 64 tokens)
    need = max(sum(-(-(p + d) // 64) * 64 for p, d in b) for b in plans)
    eng = engine(folder, dtype, max_tokens=need, max_slots=4)
    requests, steps, k = {}, [], 0
    for b, plan in enumerate(plans):
        seqs = []
        for i, (p, d) in enumerate(plan):
            rid = f"b{b}s{i}"
            requests[rid] = torch.randint(0, orc.cfg.vocab_size, (p + d,), generator=g).tolist()
            seqs.append((rid, p, d))
        live = list(seqs)
        entries = [{"id": rid, "tokens": requests[rid][:p], "want": [0, p - 1] if p > 1 else [0], "_start": 0}
                   for rid, p, d in live]
        t = 0
        while live:
            ending = [rid for rid, p, d in live if d == t]
            steps.append({"step": k, "entries": entries, "end": ending})
            k += 1
            live = [(rid, p, d) for rid, p, d in live if d > t]
            entries = [{"id": rid, "tokens": [requests[rid][p + t]], "want": [0], "_start": p + t}
                       for rid, p, d in live]
            t += 1
    got = run_trace(eng, steps, tmp_path)
    check(got, orc, requests, TOL[dtype])
    assert eng.cache.pages_in_use() == [0] * len(eng.cache.groups) and eng.cache.slots.available == 4


def test_padding_rows_change_nothing(model, tmp_path):
    name, folder, orc, prompts = model
    outs = []
    for mult in (1, 16):
        eng = engine(folder, "float32", row_multiple=mult)
        slots = [eng.open() for _ in prompts[:3]]
        a = eng.step(list(zip(slots, prompts[:3])), want="all")
        b = eng.step([(s, [7]) for s in slots], want="last")
        outs.append((a.clone(), b.clone()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


def test_a_reused_slot_holds_nothing_of_its_last_owner(model):
    name, folder, orc, prompts = model
    eng = engine(folder, "float32", max_tokens=64 * 3, max_slots=1)
    long_one = random_prompts(orc.cfg.vocab_size, [150], seed=3)[0]
    s = eng.open()
    eng.step([(s, long_one)], want=None)
    eng.close(s)
    s2 = eng.open()
    assert s2 == s
    got = eng.step([(s2, prompts[1])], want="all")
    assert max_err(got, orc.logits(prompts[1])) < TOL["float32"]


def test_trace_run_as_a_program(tmp_path):
    folder = make_folder(tmp_path, "A")
    orc = Oracle(folder)
    toks = random_prompts(orc.cfg.vocab_size, [6, 3], seed=2)
    steps = [
        {"step": 0, "entries": [{"id": "x", "tokens": toks[0][:4], "want": [3]},
                                {"id": "y", "tokens": toks[1][:2], "want": [0, 1]}], "end": []},
        {"step": 1, "entries": [{"id": "x", "tokens": [toks[0][4]], "want": [0]},
                                {"id": "y", "tokens": [toks[1][2]], "want": [0]}], "end": ["y"]},
        {"step": 2, "entries": [{"id": "x", "tokens": [toks[0][5]], "want": [0]}], "end": ["x"]},
    ]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    for dtype in ("float32", "bfloat16"):
        p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                            "--out", str(out), "--max-tokens", "128"],
                           input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                           timeout=600)
        assert p.returncode == 0, p.stderr
        assert p.stdout.split() == ["done", "0", "done", "1", "done", "2"]
        V = orc.cfg.vocab_size
        s0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(3, V)
        s2 = np.fromfile(out / "2.f32", dtype="<f4").reshape(1, V)
        tol = TOL[dtype]
        assert max_err(torch.from_numpy(s0[0]), orc.logits(toks[0])[3]) < tol
        assert max_err(torch.from_numpy(s0[2]), orc.logits(toks[1])[1]) < tol
        assert max_err(torch.from_numpy(s2[0]), orc.logits(toks[0])[5]) < tol


def test_fused_and_unfused_reduces_agree(model):
    """Steps of a few tokens leave the adding-up of their stream-k products to the next norm
    and to the rotary encoding; switching that off must give the same logits.  The same steps with
    the norms' scales applied by the norms themselves (`scaled_norm=False`) round once at another
    place: the same logits within the bfloat16 tolerance, and again the same with and without fusing."""
    name, folder, orc, prompts = model
    outs = {}
    for scaled in (True, False):
        for fuse in (True, False):
            eng = engine(folder, "bfloat16", fuse_reduce=fuse, scaled_norm=scaled, use_graphs=False)
            slots = [eng.open() for _ in prompts[:3]]
            a = eng.step(list(zip(slots, prompts[:3])), want="last")
            b = eng.step([(s, [7]) for s in slots], want="last")
            c = eng.step([(s, [9, 11]) for s in slots], want="all")
            outs[scaled, fuse] = torch.cat([a, b, c]).clone()
            eng.check()
        assert (outs[scaled, True] - outs[scaled, False]).abs().max().item() < 1e-6
    assert 0 < (outs[True, True] - outs[False, True]).abs().max().item() < TOL["bfloat16"]
    want = torch.stack([orc.logits(p + [7])[-1] for p in prompts[:3]])
    for scaled in (True, False):
        assert max_err(outs[scaled, True][3:6], want) < TOL["bfloat16"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_dump_of_the_residual_stream_after_every_layer(dtype, tmp_path):
    """`bin/trace_run --dump-activations`: a prompt in one step, then two single tokens (which
    would run through a CUDA graph without the dump); the residual stream after the embedding
    and after every layer equals the plain implementation's, and the logits are the ones a
    run without the dump writes."""
    import plain_mistral as P
    folder = sharpen(make_folder(tmp_path, "C"), 5.0)
    orc = Oracle(folder)
    toks = random_prompts(orc.cfg.vocab_size, [80], seed=9)[0]
    other = random_prompts(orc.cfg.vocab_size, [7], seed=10)[0]
    lines = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:70], "want": [69]},
                                     {"id": "b", "tokens": other[:5], "want": []}], "end": []}]
    for k in range(2):
        lines.append({"step": k + 1, "entries": [{"id": "a", "tokens": [toks[70 + k]], "want": [0]},
                                                 {"id": "b", "tokens": [other[5 + k]], "want": [0]}], "end": []})
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out, out2, acts = str(tmp_path / "out"), str(tmp_path / "out2"), str(tmp_path / "acts")
    text = "".join(json.dumps(l) + "\n" for l in lines)
    for extra, o in ((["--dump-activations", acts], out), ([], out2)):
        p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                            "--out", o, "--max-tokens", "256"] + extra, input=text, capture_output=True, text=True,
                           timeout=600)
        assert p.returncode == 0, p.stderr
        assert p.stdout.split("\n")[:3] == ["done 0", "done 1", "done 2"]
    hid_a, hid_b = [], []
    P.forward_logits(orc.w, orc.cfg, toks[:72], torch.float64, hidden=hid_a)
    P.forward_logits(orc.w, orc.cfg, other[:7], torch.float64, hidden=hid_b)
    width, runs = orc.cfg.hidden_size, orc.cfg.num_hidden_layers
    tol = 2e-5 if dtype == "float32" else 4e-2                # the stream itself, of order 1, not logits
    a0 = np.fromfile(os.path.join(acts, "0.act.f32"), dtype="<f4").reshape(1 + runs, 75, width)
    for i in range(1 + runs):
        assert np.abs(a0[i, :70] - hid_a[i][:70].numpy()).max() < tol, i
        assert np.abs(a0[i, 70:] - hid_b[i][:5].numpy()).max() < tol, i
    for k in range(2):
        ak = np.fromfile(os.path.join(acts, f"{k + 1}.act.f32"), dtype="<f4").reshape(1 + runs, 2, width)
        for i in range(1 + runs):
            assert np.abs(ak[i, 0] - hid_a[i][70 + k].numpy()).max() < tol
            assert np.abs(ak[i, 1] - hid_b[i][5 + k].numpy()).max() < tol
    for s in range(3):                                        # the dump changes no logit beyond rounding
        x = np.fromfile(os.path.join(out, f"{s}.f32"), dtype="<f4")
        y = np.fromfile(os.path.join(out2, f"{s}.f32"), dtype="<f4")
        assert x.shape == y.shape and np.abs(x - y).max() < (1e-5 if dtype == "float32" else 2e-2)
