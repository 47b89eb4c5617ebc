"""Schedules of work that the other files do not reach, against the plain implementation:
one-token steps through CUDA graphs far past the first page-table width (new graphs, new
table offsets and a new slicing of the context appear at 512 and 1,024 cached tokens), the
same steps launched kernel by kernel (bit for bit the same), one layer at the measured
model's real widths, and temperature sampling in bfloat16 through the pipelined loop."""
import math

import pytest
import torch

import plain_mistral as P
import braidinfer_b200 as lib
from braidinfer_b200.sampling import SamplingParams, uniform
from gpu_util import TOL, Oracle, engine, max_err, sharpen
from tiny import make_folder, random_prompts

pytestmark = pytest.mark.gpu


def decode_far(folder, dtype, toks, prompt_len, use_graphs):
    eng = engine(folder, dtype, max_tokens=64 * 18, max_slots=2, use_graphs=use_graphs)
    s = eng.open()
    out = [eng.step([(s, toks[:prompt_len])], want="last")]
    for t in toks[prompt_len:]:
        out.append(eng.step([(s, [t])], want="last"))
    eng.check()
    return eng, torch.cat(out)            # row i: the logits after token prompt_len - 1 + i


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_steps_past_the_first_table_widths(name, dtype, tmp_path):
    """A 40-token prompt, then one token a step up to 1,100 cached tokens.  The page tables of
    graph steps are 8, 16 and 32 columns wide in turn; every 37th logit, and every logit within
    two steps of 512 and of 1,024 cached tokens, is compared with the plain implementation, and
    the whole run must equal, bit for bit, the same run launched kernel by kernel."""
    folder = sharpen(make_folder(tmp_path, name), 6.0)
    orc = Oracle(folder)
    n, first = 1100, 40
    toks = random_prompts(orc.cfg.vocab_size, [n], seed=12)[0]
    eng, with_graphs = decode_far(folder, dtype, toks, first, True)
    assert eng.graph_replays > n - first - 10 and len(eng._graphs) >= 3        # 8, 16 and 32 columns
    want = orc.logits(toks)
    places = sorted(set(range(first - 1, n, 37)) | {p for c in (512, 1024) for p in range(c - 3, c + 3)} | {n - 1})
    worst = max(max_err(with_graphs[p - (first - 1)], want[p]) for p in places)
    assert worst < TOL[dtype], worst
    eng2, without = decode_far(folder, dtype, toks, first, False)
    assert eng2.graph_replays == 0
    assert torch.equal(with_graphs, without)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_short_prompts_through_graphs(dtype, tmp_path):
    """Steps of up to 256 tokens are given a shape (rows padded to a token tile, tables widened) and replayed
    from CUDA graphs from the third step of a shape on.  Three rounds of the same shapes with other tokens:
    two unequal prompts in one step, then a chunk that continues each, then single tokens, then three tokens each; every logit
    beside the plain implementation, and the same bits as the steps launched kernel by kernel."""
    folder = sharpen(make_folder(tmp_path, "B"), 4.0)
    orc = Oracle(folder)
    results = {}
    for use_graphs in (True, False):
        eng = engine(folder, dtype, max_tokens=64 * 24, max_slots=4, use_graphs=use_graphs)
        outs = []
        for rnd in range(3):
            seqs = random_prompts(orc.cfg.vocab_size, [33 + 9 + 2 + 3, 7 + 20 + 2 + 3], seed=40 + rnd)
            cuts = [(33, 9), (7, 20)]
            slots = [eng.open() for _ in seqs]
            a = eng.step([(sl, s[:c[0]]) for sl, s, c in zip(slots, seqs, cuts)], want="all")
            b = eng.step([(sl, s[c[0]:c[0] + c[1]]) for sl, s, c in zip(slots, seqs, cuts)], want="last")
            c1 = eng.step([(sl, [s[c[0] + c[1]]]) for sl, s, c in zip(slots, seqs, cuts)], want="last")
            c2 = eng.step([(sl, [s[c[0] + c[1] + 1]]) for sl, s, c in zip(slots, seqs, cuts)], want="last")
            # three tokens a sequence: few enough for the attention kernel that slices the context
            f = eng.step([(sl, s[c[0] + c[1] + 2:]) for sl, s, c in zip(slots, seqs, cuts)], want="all")
            eng.check()
            want = [orc.logits(s) for s in seqs]
            assert max_err(a[:33], want[0][:33]) < TOL[dtype] and max_err(a[33:], want[1][:7]) < TOL[dtype]
            assert max_err(f[:3], want[0][-3:]) < TOL[dtype] and max_err(f[3:], want[1][-3:]) < TOL[dtype]
            for j, (s, c) in enumerate(zip(seqs, cuts)):
                assert max_err(b[j], want[j][c[0] + c[1] - 1]) < TOL[dtype]
                assert max_err(c1[j], want[j][c[0] + c[1]]) < TOL[dtype]
                assert max_err(c2[j], want[j][c[0] + c[1] + 1]) < TOL[dtype]
            outs.append(torch.cat([a, b, c1, c2, f]).clone())
            for sl in slots:
                eng.close(sl)
        results[use_graphs] = torch.cat(outs)
        if use_graphs:
            assert eng.graph_replays >= 3          # the third round's prompt steps and single tokens at least
        else:
            assert eng.graph_replays == 0
    assert torch.equal(results[True], results[False])


WIDE = {
    # the measured model's layer: width 4096, 32 query and 8 kv heads of 128, feed-forward 14336
    "7b": dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=14336,
               vocab_size=2048, rope_theta=1e6, rms_norm_eps=1e-5, sliding_window=None),
    # a width that is not heads x head size (5120 against 32 x 128), and a window that the prompts run past
    "12b_window": dict(hidden_size=5120, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                       intermediate_size=14336, vocab_size=3000, rope_theta=1e6, rms_norm_eps=1e-5, sliding_window=40),
}


@pytest.mark.parametrize("name", sorted(WIDE))
def test_one_layer_at_real_widths(name):
    """The tile sizes, the stream-k plans and the attention kernels that the measured models run, met by
    float64: three unequal prompts in one step, then six single tokens each."""
    from braidinfer_b200.engine import Engine
    from braidinfer_b200.models import architecture_for
    from braidinfer_b200.weights import draw_tensors, tensor_specs_of
    d = dict(WIDE[name], architectures=["MistralForCausalLM"], num_hidden_layers=1, tie_word_embeddings=False,
             max_position_embeddings=4096)
    arch = architecture_for(d)
    drawn = draw_tensors(tensor_specs_of(arch.build_spec(arch.config_from_dict(d))), 5, torch.bfloat16)
    eng = Engine(d, {n: t.to("cuda:0") for n, t in drawn.items()}, dtype="bfloat16", max_tokens=64 * 6, max_slots=3,
                 verbose=False)
    cfg = P.PlainConfig(d)
    w64 = {n: t.double() for n, t in drawn.items()}
    del drawn
    steps = 6
    seqs = random_prompts(cfg.vocab_size, [90 + steps, 7 + steps, 33 + steps], seed=2)
    want = [P.forward_logits(w64, cfg, s, torch.float64) for s in seqs]
    cut = [90, 7, 33]
    slots = [eng.open() for _ in seqs]
    got = eng.step([(sl, s[:c]) for sl, s, c in zip(slots, seqs, cut)], want="all")
    worst, off = 0.0, 0
    for wl, c in zip(want, cut):
        worst = max(worst, max_err(got[off:off + c], wl[:c]))
        off += c
    for t in range(steps):
        out = eng.step([(sl, [s[c + t]]) for sl, s, c in zip(slots, seqs, cut)], want="last")
        for j in range(3):
            worst = max(worst, max_err(out[j], want[j][cut[j] + t]))
    eng.check()
    scale = max(1.0, max(wl.abs().max().item() for wl in want))
    assert worst < TOL["bfloat16"] * scale, (worst, scale)


def cdf_interval(logits, token, temperature, top_k):
    """[lo, hi]: the uniform numbers for which the plain chain (temperature, top-k, softmax,
    inverse CDF in index order; crates/braidinfer-runtime/src/sampling.rs:82-104, 153-170)
    picks `token`.  Empty (lo > hi) when top-k drops it."""
    x = logits.double() / temperature
    if 0 < top_k < x.numel():
        order = torch.argsort(x, descending=True, stable=True)
        x[order[top_k:]] = float("-inf")
    p = torch.softmax(x, 0)
    c = torch.cumsum(p, 0)
    return (c[token] - p[token]).item(), (c[token].item() if p[token] > 0 else -1.0)


def test_temperature_sampling_in_bfloat16_through_the_pipelined_loop(tmp_path):
    """Vocabulary 6,011, bfloat16, the loop that keeps chosen tokens on the device.  bfloat16
    logits differ from the plain ones by up to the logit tolerance e, which moves every
    cumulative probability by at most exp(2e) - 1; the uniform number of each draw must lie that
    close to the interval in which the plain chain picks the token the engine chose."""
    folder = make_folder(tmp_path, "A", vocab_size=6011)
    orc = Oracle(folder)
    prompts = random_prompts(orc.cfg.vocab_size, [5, 9, 2, 30], seed=23)
    m = lib.load(folder, dtype="bfloat16", max_seq_len=128, max_batch=4, verbose=False)
    sp = SamplingParams(temperature=0.8, seed=11)
    outs = m.generate(prompts, sp, stop_tokens=(), max_new_tokens=12)
    again = m.generate(prompts, sp, stop_tokens=(), max_new_tokens=12)
    assert [o.tokens for o in outs] == [o.tokens for o in again]
    slack = math.exp(2 * TOL["bfloat16"] / 0.8) - 1 + 0.01          # logits are divided by the temperature first
    distinct = set()
    for i, (p, o) in enumerate(zip(prompts, outs)):
        toks = list(p)
        assert len(o.tokens) == 12
        for step, t in enumerate(o.tokens):
            lo, hi = cdf_interval(orc.logits(toks)[-1], t, 0.8, 50)
            u = uniform(11, i, step)
            assert lo - slack <= u <= hi + slack, (i, step, t, u, lo, hi)
            toks.append(t)
            distinct.add(t)
    assert len(distinct) > 20                # 48 draws over 50 candidates each: not one token over and over


def test_a_requests_draws_depend_on_its_place_in_the_request_list_only(tmp_path):
    """The uniform number of a draw is a function of (seed, index of the request in the call's
    list, step).  So a request keeps its tokens when its neighbours change, and when the list is
    cut into other batches, as long as it stands at the same index."""
    folder = make_folder(tmp_path, "A")
    vocab = Oracle(folder).cfg.vocab_size
    prompts = random_prompts(vocab, [5, 9, 2, 7], seed=21)
    others = random_prompts(vocab, [3, 11, 6], seed=22)
    sp = SamplingParams(temperature=0.9, seed=4)
    m4 = lib.load(folder, dtype="float32", max_seq_len=128, max_batch=4, verbose=False)
    base = m4.generate(prompts, sp, stop_tokens=(), max_new_tokens=8)
    # other neighbours, same index
    swapped = m4.generate([others[0], prompts[1], others[2]], sp, stop_tokens=(), max_new_tokens=8)
    assert swapped[1].tokens == base[1].tokens
    assert swapped[0].tokens != base[0].tokens
    # the same list cut into batches of two, and run one request at a time: other batches, same indices
    for mb in (2, 1):
        m = lib.load(folder, dtype="float32", max_seq_len=128, max_batch=mb, verbose=False)
        cut = m.generate(prompts, sp, stop_tokens=(), max_new_tokens=8)
        assert m.last_stats.batches == 4 // mb
        assert [o.tokens for o in cut] == [o.tokens for o in base]
    # at another index the same prompt draws other numbers
    moved = m4.generate([prompts[1], prompts[0]], sp, stop_tokens=(), max_new_tokens=8)
    assert moved[0].tokens != base[1].tokens
