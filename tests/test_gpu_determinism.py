"""The same requests give the same bits every time.  Kernels here hand work from warp to warp and CTA
to CTA through barriers and partial sums; a fault in that hand-over shows as a result that changes from
run to run long before it shows against a tolerance.  Each case runs the same batch many times, with
other GPU work thrown in between to shift the timing, and compares all logits bit for bit."""
import pytest
import torch

from braidinfer_b200.engine import Engine

pytestmark = pytest.mark.gpu


def mistral(**kw):
    d = {"architectures": ["MistralForCausalLM"], "model_type": "mistral", "tie_word_embeddings": False,
         "rms_norm_eps": 1e-5, "max_position_embeddings": 32768}
    d.update(kw)
    return d


CASES = [
    # sequences of very unequal lengths, a window, 7B layer sizes: prompt kernels and decode kernels
    ("7b_window", mistral(num_hidden_layers=2, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                          head_dim=128, intermediate_size=14336, vocab_size=32000, rope_theta=10000.0,
                          sliding_window=160), [500, 37, 260], 6, 40),
    # head size 64, more sequences, no window, a long context for the sliced decode attention
    ("hd64", mistral(num_hidden_layers=2, hidden_size=1024, num_attention_heads=16, num_key_value_heads=4,
                     head_dim=64, intermediate_size=2816, vocab_size=5000, rope_theta=1e6, sliding_window=None),
     [1200, 3, 700, 64, 65], 6, 30),
    # a head size only the mma.sync kernels take, sizes that are no power of two
    ("hd48", mistral(num_hidden_layers=3, hidden_size=336, num_attention_heads=7, num_key_value_heads=7,
                     head_dim=48, intermediate_size=1000, vocab_size=3001, rope_theta=5e4, sliding_window=90),
     [300, 17, 129], 6, 30),
]


@pytest.mark.parametrize("name, cfg, lens, n_decode, repeats", CASES)
def test_the_same_batch_gives_the_same_bits(name, cfg, lens, n_decode, repeats):
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    forced = [torch.randint(0, cfg["vocab_size"], (n_decode,), generator=g).tolist() for _ in lens]
    eng = Engine.from_random(cfg, seed=3, dtype="bfloat16", on_device=True, max_tokens=64 * 48, max_slots=8, verbose=False)
    junk = torch.randn(1536, 1536, device="cuda")
    first = None
    for it in range(repeats):
        slots = [eng.open() for _ in prompts]
        if it % 3 == 1:
            junk @ junk
        outs = [eng.step(list(zip(slots, prompts)), want="last")]
        for t in range(n_decode):
            if it % 3 == 2 and t == 2:
                junk @ junk
            outs.append(eng.step([(s, [forced[i][t]]) for i, s in enumerate(slots)], want="last"))
        for s in slots:
            eng.close(s)
        got = torch.cat(outs).float().cpu()
        if first is None:
            first = got
        else:
            differ = (got != first).any(dim=1).nonzero().flatten().tolist()
            assert not differ, f"run {it}: rows {differ[:12]} of {got.shape[0]} differ from run 0 ({len(lens)} sequences a step)"
    eng.check()


def test_results_do_not_depend_on_what_lay_in_memory_before():
    """Device memory handed out by `torch.empty` holds whatever was there.  Here it holds NaN: a few
    GB are filled with NaN and given back to the allocator before the engines are built, so a kernel
    that reads a buffer (workspace, padding row, cache page) before anything wrote it shows as NaN or
    as a difference from the plain kernels."""
    blocks = [torch.full((1 << 28,), float("nan"), device="cuda", dtype=torch.float32) for _ in range(4)]
    del blocks
    name, cfg, lens, n_decode, _ = CASES[0]
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    forced = [torch.randint(0, cfg["vocab_size"], (n_decode,), generator=g).tolist() for _ in lens]
    results = []
    for backends in (dict(gemm_backend="auto", attention_backend="auto"),
                     dict(gemm_backend="plain", attention_backend="plain")):
        eng = Engine.from_random(cfg, seed=1, dtype="bfloat16", on_device=True, max_tokens=64 * 40, max_slots=4,
                                 verbose=False, **backends)
        slots = [eng.open() for _ in prompts]
        outs = [eng.step(list(zip(slots, prompts)), want="last")]
        for t in range(n_decode):
            outs.append(eng.step([(s, [forced[i][t]]) for i, s in enumerate(slots)], want="last"))
        eng.check()
        results.append(torch.cat(outs).float().cpu())
        del eng
        torch.cuda.empty_cache()
    fast, plain = results
    assert not torch.isnan(fast).any() and not torch.isnan(plain).any()
    assert (fast - plain).abs().max().item() < 2e-2 * plain.abs().max().item()
