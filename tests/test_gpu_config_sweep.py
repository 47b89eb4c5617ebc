"""Many small configurations, each different, against the plain implementation: head sizes
from 16 to 128 (64 and 128 take the tcgen05 prompt attention), one to seven heads a group,
multi-query and multi-head, widths that the tensor-core product cannot address (so the
plain product and the stacked gate/up layout run inside a bfloat16 engine), windows from 1
to beyond the context, tied and untied heads, both rotary pairings."""
import json
import os

import pytest
import torch

from gpu_util import TOL, Oracle, engine, max_err, sharpen
from tiny import random_prompts
from braidinfer_b200.weights import write_random_model

pytestmark = pytest.mark.gpu


def cfg(**kw):
    d = {"architectures": ["MistralForCausalLM"], "model_type": "mistral", "torch_dtype": "bfloat16",
         "max_position_embeddings": 2048, "tie_word_embeddings": False, "rope_theta": 10000.0,
         "rms_norm_eps": 1e-5, "sliding_window": None}
    d.update(kw)
    return d


SWEEP = {
    "hd64_gqa4": cfg(num_hidden_layers=2, hidden_size=128, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
                     intermediate_size=320, vocab_size=500),
    "hd128_mqa_window": cfg(num_hidden_layers=2, hidden_size=192, num_attention_heads=4, num_key_value_heads=1,
                            head_dim=128, intermediate_size=272, vocab_size=777, sliding_window=50, rope_theta=5e5,
                            rms_norm_eps=1e-6),
    "hd128_mha_adjacent": cfg(num_hidden_layers=1, hidden_size=256, num_attention_heads=2, num_key_value_heads=2,
                              head_dim=128, intermediate_size=130, vocab_size=260, rope_pairing="adjacent",
                              tie_word_embeddings=True),
    "hd64_group3_window1": cfg(num_hidden_layers=2, hidden_size=96, num_attention_heads=6, num_key_value_heads=2,
                               head_dim=64, intermediate_size=200, vocab_size=311, sliding_window=1),
    "hd80_group7": cfg(num_hidden_layers=1, hidden_size=112, num_attention_heads=7, num_key_value_heads=1, head_dim=80,
                       intermediate_size=96, vocab_size=129, sliding_window=3000),
    "width_not_multiple_of_8": cfg(num_hidden_layers=2, hidden_size=100, num_attention_heads=5, num_key_value_heads=5,
                                   head_dim=20, intermediate_size=70, vocab_size=203, rms_norm_eps=2e-5),
    "hd112_mixed_layers": cfg(num_hidden_layers=3, hidden_size=224, num_attention_heads=2, num_key_value_heads=1,
                              head_dim=112, intermediate_size=48, vocab_size=1000, sliding_window=33,
                              layer_types=["sliding_attention", "full_attention", "sliding_attention"]),
    "hd256": cfg(num_hidden_layers=1, hidden_size=64, num_attention_heads=2, num_key_value_heads=1, head_dim=256,
                 intermediate_size=64, vocab_size=300, rope_theta=1e6),
}


@pytest.mark.parametrize("name", sorted(SWEEP))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_configuration(name, dtype, tmp_path):
    folder = str(tmp_path / name)
    write_random_model(SWEEP[name], folder, seed=len(name))
    sharpen(folder, 4.0)
    orc = Oracle(folder)
    prompts = random_prompts(orc.cfg.vocab_size, [150, 3, 70], seed=5)
    eng = engine(folder, dtype, max_tokens=64 * 8)
    slots = [eng.open() for _ in prompts]
    cut = [140, 1, 64]
    got = eng.step([(s, p[:c]) for s, p, c in zip(slots, prompts, cut)], want="all")
    worst, off = 0.0, 0
    for p, c in zip(prompts, cut):
        worst = max(worst, max_err(got[off:off + c], orc.logits(p)[:c]))
        off += c
    for t in range(max(len(p) - c for p, c in zip(prompts, cut))):
        live = [i for i in range(3) if cut[i] + t < len(prompts[i])]
        out = eng.step([(slots[i], [prompts[i][cut[i] + t]]) for i in live], want="last")
        for j, i in enumerate(live):
            worst = max(worst, max_err(out[j], orc.logits(prompts[i])[cut[i] + t]))
    eng.check()
    # TOL is an absolute bound for logits of order 0.5; a tied head gives logits of several units
    # (a token's own embedding), and bfloat16 rounding grows with the value, so the bound scales
    scale = max(1.0, max(orc.logits(p).abs().max().item() for p in prompts))
    assert worst < TOL[dtype] * scale, (worst, scale)
