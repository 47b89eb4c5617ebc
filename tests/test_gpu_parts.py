"""Each part alone against its plain function: norm, position encoding, attention
mixer, feed-forward, embedding and head, and a block; and a schedule that names a
layer twice and lets a run read another run's cache."""
import math

import pytest
import torch

import plain_mistral as P
from braidinfer_b200.cache import CacheManager
from braidinfer_b200.csrc.api import get_kernels
from braidinfer_b200.engine.step import StepPacker
from braidinfer_b200.parts import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS,
                                   PartSpec, Runtime)
from braidinfer_b200.parts.spec import LayerSpec, ModelSpec, ScheduleEntry

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
TOLS = {torch.float32: 2e-5, torch.bfloat16: 2e-2}      # relative to the largest value compared


def close(got, want, dtype, factor=1.0):
    want = want.double().cpu()
    err = (got.double().cpu() - want).abs().max().item()
    return err < TOLS[dtype] * factor * max(1.0, want.abs().max().item())


def runtime(dtype, **kw):
    return Runtime(act_dtype=dtype, device=DEV, kernels=get_kernels(verbose=False), **kw)


def draw(part, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, ts in part.tensor_specs().items():
        x = torch.randn(ts.shape, generator=g) * (0.1 if ts.init == "normal" else 0.05)
        if ts.init == "one_plus_normal":
            x = x + 1
        out[name] = x.bfloat16().to(dtype).to(DEV)        # bfloat16 values in either run type
    return out


def step_for(mixer, seqs, dtype):
    """Cache and step context for `seqs` = [(tokens already cached, new tokens)], with the
    cached tokens' keys and values to be written by an earlier call of the mixer."""
    plan = [(mixer.cache_request(), None, mixer.state_bytes())]
    cache = CacheManager(plan, max_tokens=64 * 8, max_slots=4, dtype=dtype, device=DEV)
    return cache, StepPacker(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    rt = runtime(dtype)
    part = NORMS.get("rmsnorm")({"width": 200, "eps": 2e-6, "name": "n.weight"}, "pre.", rt)
    assert list(part.tensor_specs()) == ["pre.n.weight"]
    w = draw(part, dtype)
    part.load(w)
    h = torch.randn(6, 200, device=DEV) * 2
    out = part.forward(h)
    ref = P.rmsnorm(h.double().cpu(), w["pre.n.weight"].double().cpu(), 2e-6)
    assert out.dtype == dtype and close(out, ref, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    rt = runtime(dtype)
    part = FEED_FORWARDS.get("swiglu")({"hidden_size": 72, "intermediate_size": 200}, "L.", rt)
    assert sorted(part.tensor_specs()) == ["L.mlp.down_proj.weight", "L.mlp.gate_proj.weight", "L.mlp.up_proj.weight"]
    w = draw(part, dtype)
    part.load(w)
    x = (torch.randn(9, 72, device=DEV)).to(dtype)
    res = torch.randn(9, 72, device=DEV)
    want = res.double().cpu() + P.swiglu(x.double().cpu(), w["L.mlp.gate_proj.weight"].double().cpu(),
                                         w["L.mlp.up_proj.weight"].double().cpu(),
                                         w["L.mlp.down_proj.weight"].double().cpu())
    got = part.forward(x, res, None)
    assert got.dtype == torch.float32 and close(got, want, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_head_parts(dtype):
    rt = runtime(dtype)
    emb = EMBEDDINGS.get("token_embedding")({"vocab_size": 77, "hidden_size": 40}, "", rt)
    w = draw(emb, dtype)
    emb.load(w)
    ids = torch.tensor([3, 76, 0], dtype=torch.int32, device=DEV)
    h = emb.forward(ids, 3)
    assert torch.equal(h.cpu(), w["model.embed_tokens.weight"].float().cpu()[[3, 76, 0]])
    head = HEADS.get("linear_head")({"vocab_size": 77, "hidden_size": 40, "tied": True}, "", rt)
    assert head.tensor_specs() == {}
    head.load({})
    head.tie(emb.weight)
    x = torch.randn(3, 40, device=DEV).to(dtype)
    lg = head.forward(x)
    ref = P.linear(x.double().cpu(), w["model.embed_tokens.weight"].double().cpu())
    assert lg.dtype == torch.float32 and close(lg, ref, dtype)


def attention_params(window, pairing):
    rope = PartSpec("rope", {"head_dim": 32, "theta": 5e4, "rope_dim": 32, "pairing": pairing})
    return {"hidden_size": 72, "num_heads": 6, "num_kv_heads": 3, "head_dim": 32, "window": window,
            "position_encoding": rope}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window, pairing", [(None, "half"), (5, "adjacent")])
def test_attention_mixer_part(dtype, window, pairing):
    rt = runtime(dtype)
    mixer = MIXERS.get("gqa_attention")(attention_params(window, pairing), "L.", rt)
    req = mixer.cache_request()
    assert (req.kind, req.num_kv_heads, req.head_dim, req.window) == ("window" if window else "full", 3, 32, window)
    w = draw(mixer, dtype)
    mixer.load(w)
    cache, packer = step_for(mixer, None, dtype)
    T = 70
    x = (torch.randn(T, 72, device=DEV) * 2).to(dtype)
    res = torch.randn(T, 72, device=DEV)
    # plain: the same maths on the whole sequence
    class Cfg:
        num_attention_heads, num_key_value_heads, head_dim = 6, 3, 32
        rope_theta, rope_pairing, rms_norm_eps = 5e4, pairing, 1e-5
        @staticmethod
        def layer_window(i):
            return window
    wd = {k: v.double().cpu() for k, v in w.items()}
    xd = x.double().cpu()
    q = P.rope(P.linear(xd, wd["L.self_attn.q_proj.weight"]).view(T, 6, 32), torch.arange(T), 5e4, pairing)
    k = P.rope(P.linear(xd, wd["L.self_attn.k_proj.weight"]).view(T, 3, 32), torch.arange(T), 5e4, pairing)
    v = P.linear(xd, wd["L.self_attn.v_proj.weight"]).view(T, 3, 32)
    want = res.double().cpu() + P.linear(P.attention(q, k, v, window).reshape(T, 192), wd["L.self_attn.o_proj.weight"])
    # the part: 66 tokens in one step, then 4 one by one, through the cache
    slot = cache.alloc_slot()
    got = []
    for lo, hi in [(0, 66), (66, 67), (67, 68), (68, 69), (69, 70)]:
        tables = cache.begin_step([slot], [hi - lo])
        ctx = packer.pack([slot], [[0] * (hi - lo)], [lo], [[]], tables)
        view = cache.layer_view(0)
        view.page_table = ctx.page_tables[0]
        out = mixer.forward(x[lo:hi].contiguous(), res[lo:hi].clone(), ctx, view, None)
        got.append(ctx.resolve(out))             # the mixer may have left its last sum to the next norm
        cache.end_step([slot], [hi - lo])
    rt.kernels.check_device_errors()
    assert close(torch.cat(got), want, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_position_encoding_part_alone(dtype):
    rt = runtime(dtype)
    pe = POSITION_ENCODINGS.get("rope")({"head_dim": 16, "theta": 1e4, "rope_dim": 16, "pairing": "half"}, "", rt)
    assert torch.allclose(pe.inv_freq.cpu(), P.inv_freq(16, 1e4))
    packer = StepPacker(DEV)
    ctx = packer.pack([0], [[0, 0, 0]], [40], [[]], [])
    qkv = torch.randn(3, (2 + 2) * 16, device=DEV).to(dtype)
    before = qkv.clone()
    pe.encode_and_store(qkv, 2, 1, ctx, None)              # no cache: rotate only
    x = before.double().cpu().view(3, 4, 16)
    want = P.rope(x[:, :3].contiguous(), torch.tensor([40, 41, 42]), 1e4, "half")
    got = qkv.double().cpu().view(3, 4, 16)
    assert (got[:, :3] - want).abs().max() < (1e-5 if dtype == torch.float32 else 4e-2)
    assert torch.equal(got[:, 3], x[:, 3])


def test_block_and_schedule_against_the_plain_model(tmp_path):
    """A model description written by hand: layer 0 runs twice (each run with a cache of
    its own), and the last run of layer 1 reads the keys and values of its first run."""
    from tiny import TINY_A, make_folder, read_weights, config_of, random_prompts
    from braidinfer_b200.engine import Engine
    from braidinfer_b200.models import architecture_for
    import dataclasses
    folder = make_folder(tmp_path, "A")
    cfg = config_of(folder)
    arch = architecture_for(TINY_A)
    base = arch.build_spec(arch.config_from_dict(TINY_A))
    sched = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_of=1))
    spec = dataclasses.replace(base, schedule=sched)
    toks = random_prompts(cfg.vocab_size, [75], seed=1)[0]
    want = P.forward_logits(read_weights(folder), cfg, toks, torch.float64,
                            schedule=[(0, None), (1, None), (0, None), (1, 1)])
    from braidinfer_b200.weights import load_tensors, tensor_specs_of
    for dtype in ("float32", "bfloat16"):
        run_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
        tensors = load_tensors(folder, tensor_specs_of(spec), run_dtype, "cuda:0")
        eng = Engine(None, tensors, spec=spec, dtype=dtype, max_tokens=256, max_slots=4, verbose=False)
        assert eng.cache.groups[0].storage.shape[0] == 3          # three runs keep a cache, one borrows
        s = eng.open()
        got = [eng.step([(s, toks[:70])], want="all")] + [eng.step([(s, [t])], want="last") for t in toks[70:]]
        eng.check()
        err = (torch.cat(got).double().cpu() - want).abs().max().item()
        assert err < (2e-5 if dtype == "float32" else 1.5e-2), err
