"""The plain implementation checked against hand-worked numbers and against properties
that follow from the formulas (CPU)."""
import math

import pytest
import torch

import plain_mistral as P
from braidinfer_b200.config import MistralConfig
from braidinfer_b200.weights import draw_tensors, tensor_specs_of
from braidinfer_b200.models import architecture_for
from tiny import TINY_A, TINY_B, TINY_C


def test_rmsnorm_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    r = 1.0 / math.sqrt((9 + 16) / 2 + 1e-5)
    assert torch.allclose(P.rmsnorm(x, w, 1e-5), torch.tensor([[3 * r * 2, 4 * r * 0.5]], dtype=torch.float64))


def test_inv_freq_and_rotation_by_hand():
    f = P.inv_freq(4, 100.0, torch.float64)
    assert torch.allclose(f, torch.tensor([1.0, 0.1], dtype=torch.float64))
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]], dtype=torch.float64)
    pos = torch.tensor([2])
    adj = P.rope(x, pos, 100.0, "adjacent")[0, 0]
    c0, s0, c1, s1 = math.cos(2.0), math.sin(2.0), math.cos(0.2), math.sin(0.2)
    assert torch.allclose(adj, torch.tensor([1 * c0 - 2 * s0, 1 * s0 + 2 * c0, 3 * c1 - 4 * s1, 3 * s1 + 4 * c1],
                                            dtype=torch.float64))
    half = P.rope(x, pos, 100.0, "half")[0, 0]
    assert torch.allclose(half, torch.tensor([1 * c0 - 3 * s0, 2 * c1 - 4 * s1, 1 * s0 + 3 * c0, 2 * s1 + 4 * c1],
                                             dtype=torch.float64))


@pytest.mark.parametrize("pairing", ["half", "adjacent"])
def test_rotated_scores_depend_on_distance_only(pairing):
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, 1, 8, generator=g, dtype=torch.float64)
    k = torch.randn(1, 1, 8, generator=g, dtype=torch.float64)
    def score(pq, pk):
        return (P.rope(q, torch.tensor([pq]), 1e4, pairing) * P.rope(k, torch.tensor([pk]), 1e4, pairing)).sum()
    assert abs(score(5, 2) - score(105, 102)) < 1e-9
    assert abs(score(5, 2) - score(5, 3)) > 1e-6


def test_attention_mask_and_groups_by_hand():
    T, hd = 4, 2
    q = torch.zeros(T, 2, hd, dtype=torch.float64)          # zero queries: uniform over visible keys
    k = torch.randn(T, 1, hd, dtype=torch.float64)
    v = torch.arange(T, dtype=torch.float64).view(T, 1, 1).repeat(1, 1, hd)
    full = P.attention(q, k, v, None)
    assert torch.allclose(full[:, 0, 0], torch.tensor([0.0, 0.5, 1.0, 1.5], dtype=torch.float64))
    assert torch.allclose(full[:, 1], full[:, 0])           # both heads read kv head 0
    win = P.attention(q, k, v, 2)
    assert torch.allclose(win[:, 0, 0], torch.tensor([0.0, 0.5, 1.5, 2.5], dtype=torch.float64))
    one = P.attention(q, k, v, 1)
    assert torch.allclose(one[:, 0, 0], torch.tensor([0.0, 1.0, 2.0, 3.0], dtype=torch.float64))


def test_swiglu_by_hand():
    x = torch.tensor([[1.0, -2.0]], dtype=torch.float64)
    wg = torch.tensor([[1.0, 0.0]], dtype=torch.float64)
    wu = torch.tensor([[0.0, 1.0]], dtype=torch.float64)
    wd = torch.tensor([[3.0], [1.0]], dtype=torch.float64)
    a = 1.0 / (1.0 + math.exp(-1.0)) * -2.0
    assert torch.allclose(P.swiglu(x, wg, wu, wd), torch.tensor([[3 * a, a]], dtype=torch.float64))


def weights_for(d, seed):
    """Random tensors under the model's tensor names (data only) and the plain reading of the configuration."""
    arch = architecture_for(d)
    drawn = draw_tensors(tensor_specs_of(arch.build_spec(arch.config_from_dict(d))), seed)
    return P.PlainConfig(d), {n: t.double() for n, t in drawn.items()}


@pytest.mark.parametrize("d", [TINY_A, TINY_B, TINY_C,
                               {"hidden_size": 48, "num_attention_heads": 4, "intermediate_size": 100,
                                "num_hidden_layers": 2, "vocab_size": 50, "partial_rotary_factor": 0.5}])
def test_the_package_reads_config_json_as_the_plain_reader_does(d):
    """Two readings of the same keys, written apart: every size, constant and default, and each
    layer's window, must agree (a wrong default would otherwise be wrong on both sides of every test)."""
    mine, theirs = P.PlainConfig(d), MistralConfig.from_dict(dict(d, architectures=["MistralForCausalLM"]))
    for key in ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
                "intermediate_size", "vocab_size", "rms_norm_eps", "rope_theta", "rope_dim", "rope_pairing"):
        assert getattr(mine, key) == getattr(theirs, key), key
    for i in range(mine.num_hidden_layers):
        assert mine.layer_window(i) == theirs.layer_window(i), i


def test_partial_rotation_by_hand():
    # head of 6, 4 of them rotated: pairs (0, 2) and (1, 3) for "half", (0, 1) and (2, 3) for "adjacent";
    # frequencies come from the rotated size (4), elements 4 and 5 pass through
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]]], dtype=torch.float64)
    pos = torch.tensor([3])
    c0, s0, c1, s1 = math.cos(3.0), math.sin(3.0), math.cos(0.3), math.sin(0.3)
    half = P.rope(x, pos, 100.0, "half", rope_dim=4)[0, 0]
    assert torch.allclose(half, torch.tensor([1 * c0 - 3 * s0, 2 * c1 - 4 * s1, 1 * s0 + 3 * c0, 2 * s1 + 4 * c1, 5.0, 6.0],
                                             dtype=torch.float64))
    adj = P.rope(x, pos, 100.0, "adjacent", rope_dim=4)[0, 0]
    assert torch.allclose(adj, torch.tensor([1 * c0 - 2 * s0, 1 * s0 + 2 * c0, 3 * c1 - 4 * s1, 3 * s1 + 4 * c1, 5.0, 6.0],
                                            dtype=torch.float64))


def test_later_tokens_do_not_change_earlier_logits_and_window_forgets():
    cfg, w = weights_for(TINY_B, 7)
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, cfg.vocab_size, (24,), generator=g).tolist()
    full = P.forward_logits(w, cfg, toks, torch.float64)
    assert full.shape == (24, cfg.vocab_size)
    assert torch.allclose(P.forward_logits(w, cfg, toks[:10], torch.float64), full[:10], atol=1e-12)
    # 3 layers of window 8 reach back at most 3 * 7 = 21 tokens: token 0 cannot reach position 23
    other = [(toks[0] + 1) % cfg.vocab_size] + toks[1:]
    changed = P.forward_logits(w, cfg, other, torch.float64)
    assert torch.allclose(changed[23], full[23], atol=1e-12)
    assert not torch.allclose(changed[5], full[5], atol=1e-9)
    cfg_a, w_a = weights_for(TINY_A, 0)
    toks_a = [t % cfg_a.vocab_size for t in toks]
    fa = P.forward_logits(w_a, cfg_a, toks_a, torch.float64)
    other_a = [(toks_a[0] + 1) % cfg_a.vocab_size] + toks_a[1:]
    assert not torch.allclose(P.forward_logits(w_a, cfg_a, other_a, torch.float64)[23], fa[23], atol=1e-9)


def test_schedule_of_the_plain_model():
    cfg, w = weights_for(TINY_A, 0)
    toks = [5, 9, 200, 31, 7]
    base = P.forward_logits(w, cfg, toks, torch.float64)
    same = P.forward_logits(w, cfg, toks, torch.float64, schedule=[(0, None), (1, None)])
    assert torch.allclose(base, same, atol=1e-12)
    twice = P.forward_logits(w, cfg, toks, torch.float64, schedule=[(0, None), (1, None), (0, None), (1, 1)])
    assert not torch.allclose(base, twice, atol=1e-6)


def test_sampling_chain_by_hand():
    lg = torch.tensor([1.0, 3.0, 2.0, 3.0, -1.0])
    assert P.argmax_lowest(lg) == 1                                     # lowest index of a tie
    assert P.sample(lg, temperature=0.0) == 1
    assert P.sample(lg, temperature=0.0, logit_bias=[(4, 10.0)]) == 4
    # repetition penalty: positive logits are divided, negative multiplied, once per occurrence
    assert P.sample(lg, temperature=0.0, repetition_penalty=2.0, history=[1, 3, 3]) == 2
    # top_k = 1 leaves only index 1 (the tie goes to the lower index)
    for u in (1e-6, 0.5, 0.999):
        assert P.sample(lg, temperature=1.0, top_k=1, u=u) == 1
    # inverse CDF: probabilities of [0, ln 3] are [0.25, 0.75]
    two = torch.tensor([0.0, math.log(3.0)])
    assert P.sample(two, temperature=1.0, u=0.2) == 0 and P.sample(two, temperature=1.0, u=0.3) == 1
    # top_p keeps the smallest set reaching it: 0.75 >= 0.7 keeps index 1 only
    assert P.sample(two, temperature=1.0, top_p=0.7, u=0.01) == 1
    # min_p drops what is below min_p * max
    assert P.sample(two, temperature=1.0, min_p=0.5, u=0.01) == 1
    # temperature sharpens
    assert P.sample(two, temperature=0.1, u=0.001) == 1
