"""The tensor-core kernels at the sizes of real models, end to end, against the plain
kernels (FFMA product, one-warp-per-query attention) on the same weights: Mistral-7B
layer sizes with a sliding window whose pages are given back, and the Mistral-NeMo
sizes (head_dim that is not hidden / heads, a vocabulary of 131072).  A couple of layers
each, random weights, bfloat16; both engines round alike, so their logits differ by
accumulation order only."""
import pytest
import torch

from braidinfer_b200.engine import Engine

pytestmark = pytest.mark.gpu


def mistral(**kw):
    d = {"architectures": ["MistralForCausalLM"], "model_type": "mistral", "tie_word_embeddings": False,
         "rms_norm_eps": 1e-5, "max_position_embeddings": 32768}
    d.update(kw)
    return d


def run(eng, prompts, n_decode, forced):
    """Prompts in one step, then `n_decode` one-token steps of given tokens; all logits."""
    slots = [eng.open() for _ in prompts]
    out = [eng.step(list(zip(slots, prompts)), want="last")]
    for t in range(n_decode):
        out.append(eng.step([(s, [forced[i][t]]) for i, s in enumerate(slots)], want="last"))
    eng.check()
    for s in slots:
        eng.close(s)
    return torch.cat(out).float().cpu()


@pytest.mark.parametrize("name, cfg, lens, n_decode", [
    ("7b_window", mistral(num_hidden_layers=2, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                          head_dim=128, intermediate_size=14336, vocab_size=32000, rope_theta=10000.0,
                          sliding_window=160), [500, 37, 260], 40),
    # 390 and 210 rows a step: the products whose whole tiles would leave SMs idle go as partial sums
    ("7b_390_rows", mistral(num_hidden_layers=2, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                            head_dim=128, intermediate_size=14336, vocab_size=32000, rope_theta=1e6,
                            sliding_window=None), [300, 90], 6),
    ("7b_210_rows", mistral(num_hidden_layers=2, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                            head_dim=128, intermediate_size=14336, vocab_size=32000, rope_theta=1e6,
                            sliding_window=None), [120, 60, 30], 6),
    ("7b_700_rows", mistral(num_hidden_layers=2, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                            head_dim=128, intermediate_size=14336, vocab_size=32000, rope_theta=1e6,
                            sliding_window=None), [640, 60], 4),
    ("nemo", mistral(num_hidden_layers=1, hidden_size=5120, num_attention_heads=32, num_key_value_heads=8,
                     head_dim=128, intermediate_size=14336, vocab_size=131072, rope_theta=1e6,
                     sliding_window=None), [700, 33, 128, 65], 12),
])
def test_tensor_core_engine_equals_plain_engine_at_model_sizes(name, cfg, lens, n_decode):
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    forced = [torch.randint(0, cfg["vocab_size"], (n_decode,), generator=g).tolist() for _ in lens]
    results = []
    for backends in (dict(gemm_backend="auto", attention_backend="auto"),
                     dict(gemm_backend="plain", attention_backend="plain")):
        eng = Engine.from_random(cfg, seed=1, dtype="bfloat16", on_device=True, max_tokens=64 * 40, max_slots=4,
                                 verbose=False, **backends)
        results.append(run(eng, prompts, n_decode, forced))
        if cfg["sliding_window"]:
            assert eng.cache.pages_in_use() == [0]
        del eng
        torch.cuda.empty_cache()
    fast, plain = results
    scale = plain.abs().max().item()
    per_row = (fast - plain).abs().max(dim=1).values          # rows: the prompts' last tokens, then a row a sequence and step
    bad = [(i, round(v, 4)) for i, v in enumerate(per_row.tolist()) if v >= 2e-2 * scale]
    assert not bad, f"rows (index, difference) beyond {2e-2 * scale:.4f}: {bad[:16]} of {len(per_row)} rows, {len(lens)} sequences"
    # the choice of token agrees wherever the plain logits have a clear winner
    top2 = plain.topk(2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 4e-2 * scale
    assert torch.equal(fast.argmax(-1)[clear], plain.argmax(-1)[clear])


def test_window_pages_are_given_back_while_decoding():
    cfg = mistral(num_hidden_layers=1, hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                  intermediate_size=512, vocab_size=1000, rope_theta=10000.0, sliding_window=100)
    eng = Engine.from_random(cfg, seed=0, dtype="bfloat16", max_tokens=64 * 6, max_slots=1, verbose=False)
    s = eng.open()
    eng.step([(s, list(range(300)))], want=None)            # needs 5 pages during the step ...
    assert eng.cache.pages_in_use() == [2]                  # ... and keeps the 2 or 3 the window still covers
    for t in range(600):                                    # far beyond the 384 tokens the cache has room for
        eng.step([(s, [t % 1000])], want="last")
        assert eng.cache.pages_in_use()[0] <= 3
    eng.check()
    assert eng.length(s) == 900
