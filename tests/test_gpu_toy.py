"""A toy mixer with state of its own, defined here, registered, built into a model
description and stepped through the engine, without a change to the library's files.

The mixer keeps, per sequence, a running sum of its inputs (float32, fixed size) and a
count; its output for token t is W (sum of inputs up to t) / (t + 1).  It has no keys
and values, so it asks for no cache, only for state bytes.  Its forward is plain torch
on the GPU (a test may do that; the library's own parts may not) and reads the step's
host-side fields, so it marks itself as not replayable by a CUDA graph.
"""
import dataclasses

import pytest
import torch

from braidinfer_b200.parts import MIXERS, Mixer, PartSpec
from braidinfer_b200.parts.spec import LayerSpec, TensorSpec

pytestmark = pytest.mark.gpu


class RunningMeanMixer(Mixer):
    graph_safe = False

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.width = int(params["width"])
        self.name = prefix + "toy.mix.weight"

    def tensor_specs(self):
        return {self.name: TensorSpec((self.width, self.width))}

    def load(self, tensors):
        self.w = tensors[self.name].float()

    def cache_request(self):
        return None

    def state_bytes(self):
        return 4 * (self.width + 1)              # float32 running sum and a count

    def forward(self, x, residual, ctx, cache, state):
        assert cache is None and state is not None
        st = state.view(torch.float32)           # [slots, width + 1]
        out = torch.empty_like(residual)
        r = 0
        for slot, n in zip(ctx.host_slots, ctx.host_q_len):
            xs = x[r:r + n].float()
            sums = st[slot, :self.width] + torch.cumsum(xs, 0)
            counts = st[slot, self.width] + torch.arange(1, n + 1, device=x.device)
            out[r:r + n] = residual[r:r + n] + (sums / counts[:, None]) @ self.w.t()
            st[slot, :self.width] = sums[-1]
            st[slot, self.width] = counts[-1]
            r += n
        if ctx.rows > r:
            out[r:] = residual[r:]
        return out


def plain_running_mean_model(weights, cfg, tokens, eps):
    """The toy model, whole sequence, float64: layer 0 uses the toy mixer, layer 1 attention."""
    import plain_mistral as P
    w = {k: v.double() for k, v in weights.items()}
    T = len(tokens)
    h = P.embedding(w["model.embed_tokens.weight"], tokens, torch.float64)
    n = P.rmsnorm(h, w["model.layers.0.input_layernorm.weight"], eps)
    means = torch.cumsum(n, 0) / torch.arange(1, T + 1, dtype=torch.float64)[:, None]
    h = h + means @ w["model.layers.0.toy.mix.weight"].t()
    n = P.rmsnorm(h, w["model.layers.0.post_attention_layernorm.weight"], eps)
    h = h + P.swiglu(n, w["model.layers.0.mlp.gate_proj.weight"], w["model.layers.0.mlp.up_proj.weight"],
                     w["model.layers.0.mlp.down_proj.weight"])
    h = P.decoder_layer(h, w, 1, cfg, torch.arange(T))
    h = P.rmsnorm(h, w["model.norm.weight"], eps)
    return P.linear(h, w["lm_head.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_is_registered_built_and_stepped(dtype):
    from braidinfer_b200.cache import CacheManager
    from braidinfer_b200.engine import Engine
    from braidinfer_b200.models import DecoderModel, architecture_for
    from braidinfer_b200.weights import draw_tensors
    from tiny import TINY_A, random_prompts
    MIXERS.register("toy_running_mean", RunningMeanMixer)
    try:
        arch = architecture_for(TINY_A)
        cfg = arch.config_from_dict(TINY_A)
        base = arch.build_spec(cfg)
        toy_layer = dataclasses.replace(base.layers[0], mixer=PartSpec("toy_running_mean", {"width": cfg.hidden_size}))
        spec = dataclasses.replace(base, layers=(toy_layer, base.layers[1]))
        # an engine of the stock model first, then the description is swapped and rebuilt
        eng = Engine.from_random(TINY_A, 0, dtype=dtype, max_tokens=512, max_slots=3, verbose=False)
        eng.spec = spec
        eng.model = DecoderModel(spec, eng.rt)
        specs = eng.model.tensor_specs()
        assert "model.layers.0.toy.mix.weight" in specs and "model.layers.0.self_attn.q_proj.weight" not in specs
        drawn = draw_tensors(specs, 5)
        eng.model.load({n: (t.to(eng.device) if dtype == "bfloat16" else t.to(eng.device).float())
                        for n, t in drawn.items()})
        eng.cache = CacheManager(eng.model.cache_plan(), 512, 3, eng.dtype, eng.device)
        eng.use_graphs = all(p.graph_safe for p in eng.model.all_parts())
        assert eng.use_graphs is False
        assert eng.cache.state_view(0).shape == (3, 4 * (cfg.hidden_size + 1)) and eng.cache.state_view(1) is None
        assert len(eng.cache.groups) == 1 and eng.cache.groups[0].storage.shape[0] == 1     # only layer 1 keeps keys

        prompts = random_prompts(cfg.vocab_size, [9, 4, 14], seed=2)
        w64 = {n: t.double() for n, t in drawn.items()}
        want = [plain_running_mean_model(w64, cfg, p, cfg.rms_norm_eps) for p in prompts]
        tol = 2e-5 if dtype == "float32" else 1.5e-2
        # a batch of unequal prompts, then one token each; the shortest ends first; then its slot is used again
        slots = [eng.open() for _ in prompts]
        cut = [5, 2, 7]
        lg = eng.step([(s, p[:c]) for s, p, c in zip(slots, prompts, cut)], want="all")
        off = 0
        for p, c, wnt in zip(prompts, cut, want):
            assert (lg[off:off + c].double().cpu() - wnt[:c]).abs().max() < tol
            off += c
        for t in range(max(len(p) - c for p, c in zip(prompts, cut))):
            live = [i for i in range(3) if cut[i] + t < len(prompts[i])]
            lg = eng.step([(slots[i], [prompts[i][cut[i] + t]]) for i in live], want="last")
            for j, i in enumerate(live):
                assert (lg[j].double().cpu() - want[i][cut[i] + t]).abs().max() < tol
            for i in range(3):
                if cut[i] + t + 1 == len(prompts[i]):
                    eng.close(slots[i])
        s = eng.open()                           # a used slot: its state must start at zero again
        lg = eng.step([(s, prompts[0])], want="all")
        assert (lg.double().cpu() - want[0]).abs().max() < tol
    finally:
        MIXERS.unregister("toy_running_mean")
