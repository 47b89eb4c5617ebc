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
        eng = Engine.from_spec(spec, 5, dtype=dtype, max_tokens=512, max_slots=3, verbose=False)
        specs = eng.model.tensor_specs()
        assert "model.layers.0.toy.mix.weight" in specs and "model.layers.0.self_attn.q_proj.weight" not in specs
        drawn = eng.drawn
        assert eng.use_graphs is False               # the toy mixer said it cannot be replayed by a graph
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


# ---------------------------------------------------------------------------------------------
# A toy feed-forward with routing and a toy position encoding, also defined here only.
#
# The feed-forward has two experts (small two-layer perceptrons with a tanh) and a router;
# each token goes to the expert with the larger router logit (the lower index on a tie) and
# its output is weighted by the softmax probability of that expert.  The position encoding
# rotates nothing: it adds a learned vector per position (up to 256 positions) to queries
# and keys and then stores keys and values with the library's own cache-write kernel.
from braidinfer_b200.parts import FEED_FORWARDS, POSITION_ENCODINGS, FeedForward, PositionEncoding


class TopOneExperts(FeedForward):
    graph_safe = False          # it gathers rows by a data-dependent index: a CUDA graph cannot replay that

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.width, self.inner, self.n = int(params["width"]), int(params["inner"]), int(params["experts"])
        self.prefix = prefix

    def tensor_specs(self):
        d = {self.prefix + "toy.router.weight": TensorSpec((self.n, self.width))}
        for e in range(self.n):
            d[self.prefix + f"toy.experts.{e}.w1.weight"] = TensorSpec((self.inner, self.width))
            d[self.prefix + f"toy.experts.{e}.w2.weight"] = TensorSpec((self.width, self.inner))
        return d

    def load(self, tensors):
        self.router = tensors[self.prefix + "toy.router.weight"].float()
        self.w1 = [tensors[self.prefix + f"toy.experts.{e}.w1.weight"].float() for e in range(self.n)]
        self.w2 = [tensors[self.prefix + f"toy.experts.{e}.w2.weight"].float() for e in range(self.n)]

    def forward(self, x, residual, ctx):
        xf = x.float()
        logits = xf @ self.router.t()                           # router logits in float32
        prob = torch.softmax(logits, -1)
        choice = logits.argmax(-1)
        out = residual.clone()
        for e in range(self.n):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                y = torch.tanh(xf[rows] @ self.w1[e].t()) @ self.w2[e].t()
                out[rows] += prob[rows, e:e + 1] * y
        return out


class LearnedOffsets(PositionEncoding):
    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.hd, self.max_pos = int(params["head_dim"]), int(params["max_positions"])
        self.name = prefix + "toy.position.weight"
        self.zero_freq = torch.zeros(self.hd // 2, dtype=torch.float32, device=runtime.device)

    def tensor_specs(self):
        return {self.name: TensorSpec((self.max_pos, self.hd))}

    def load(self, tensors):
        self.table = tensors[self.name]

    def encode_and_store(self, qkv, nqh, nkh, ctx, cache):
        rows = ctx.n_tokens
        pos = ctx.positions[:rows].long()
        view = qkv[:rows].view(rows, nqh + 2 * nkh, self.hd)
        view[:, :nqh + nkh] += self.table[pos].to(qkv.dtype)[:, None, :]
        # angle zero: the library's kernel leaves queries and keys as they are and stores keys and values
        writable = cache is not None and not cache.read_only
        self.rt.kernels.rope_kv_write(qkv, self.zero_freq, ctx.positions, ctx.token_seq,
                                      cache.page_table if writable else None, cache.storage if writable else None,
                                      nqh, nkh, self.hd, self.hd, False, cache.page_size if cache is not None else 1)


def plain_toy_model_2(weights, cfg, tokens):
    import plain_mistral as P
    w = {k: v.double() for k, v in weights.items()}
    T = len(tokens)
    nqh, nkh, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    h = P.embedding(w["model.embed_tokens.weight"], tokens, torch.float64)
    for layer in range(cfg.num_hidden_layers):
        pre = f"model.layers.{layer}."
        n = P.rmsnorm(h, w[pre + "input_layernorm.weight"], cfg.rms_norm_eps)
        off = w[pre + "toy.position.weight"][:T]
        q = P.linear(n, w[pre + "self_attn.q_proj.weight"]).view(T, nqh, hd) + off[:, None, :]
        k = P.linear(n, w[pre + "self_attn.k_proj.weight"]).view(T, nkh, hd) + off[:, None, :]
        v = P.linear(n, w[pre + "self_attn.v_proj.weight"]).view(T, nkh, hd)
        h = h + P.linear(P.attention(q, k, v, cfg.layer_window(layer)).reshape(T, nqh * hd), w[pre + "self_attn.o_proj.weight"])
        n = P.rmsnorm(h, w[pre + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
        logits = n @ w[pre + "toy.router.weight"].t()
        prob = torch.softmax(logits, -1)
        choice = logits.argmax(-1)
        y = torch.zeros_like(h)
        for e in range(2):
            m = choice == e
            y[m] = prob[m, e:e + 1] * (torch.tanh(n[m] @ w[pre + f"toy.experts.{e}.w1.weight"].t())
                                       @ w[pre + f"toy.experts.{e}.w2.weight"].t())
        h = h + y
    h = P.rmsnorm(h, w["model.norm.weight"], cfg.rms_norm_eps)
    return P.linear(h, w["lm_head.weight"]), None


def test_toy_routed_feed_forward_and_toy_position_encoding():
    from braidinfer_b200.cache import CacheManager
    from braidinfer_b200.engine import Engine
    from braidinfer_b200.models import DecoderModel, architecture_for
    from braidinfer_b200.weights import draw_tensors
    from tiny import TINY_A, random_prompts
    FEED_FORWARDS.register("toy_top_one_experts", TopOneExperts)
    POSITION_ENCODINGS.register("toy_learned_offsets", LearnedOffsets)
    try:
        arch = architecture_for(TINY_A)
        cfg = arch.config_from_dict(TINY_A)
        base = arch.build_spec(cfg)
        layers = []
        for ls in base.layers:
            mp = dict(ls.mixer.params)
            mp["position_encoding"] = PartSpec("toy_learned_offsets", {"head_dim": cfg.head_dim, "max_positions": 256})
            layers.append(dataclasses.replace(
                ls, mixer=PartSpec("gqa_attention", mp),
                feed_forward=PartSpec("toy_top_one_experts", {"width": cfg.hidden_size, "inner": 40, "experts": 2})))
        spec = dataclasses.replace(base, layers=tuple(layers))
        # scaled so that the routing is decisive and the offsets matter
        eng = Engine.from_spec(spec, 9, dtype="float32", max_tokens=512, max_slots=3, verbose=False,
                               scale={"toy.router.weight": 20.0, "toy.position.weight": 20.0})
        specs = eng.model.tensor_specs()
        assert "model.layers.1.toy.experts.1.w2.weight" in specs and "model.layers.0.mlp.gate_proj.weight" not in specs
        drawn = eng.drawn
        assert eng.use_graphs is False
        prompts = random_prompts(cfg.vocab_size, [70, 9], seed=3)
        w64 = {n_: t.double() for n_, t in drawn.items()}
        want = [plain_toy_model_2(w64, cfg, p)[0] for p in prompts]
        slots = [eng.open() for _ in prompts]
        cut = [66, 5]
        got = eng.step([(s, p[:c]) for s, p, c in zip(slots, prompts, cut)], want="all")
        assert (got[:66].double().cpu() - want[0][:66]).abs().max() < 2e-5
        assert (got[66:].double().cpu() - want[1][:5]).abs().max() < 2e-5
        for t in range(4):
            out = eng.step([(slots[i], [prompts[i][cut[i] + t]]) for i in range(2)], want="last")
            for i in range(2):
                assert (out[i].double().cpu() - want[i][cut[i] + t]).abs().max() < 2e-5
        eng.check()
    finally:
        FEED_FORWARDS.unregister("toy_top_one_experts")
        POSITION_ENCODINGS.unregister("toy_learned_offsets")


# ---------------------------------------------------------------------------------------------
# A toy feed-forward that takes row scales: in steps of few tokens the library's norm hands it rows that
# are multiplied by the norm's weights only, and the scale that is still owed (StepContext.row_scales).
class ScaleAwarePerceptron(FeedForward):
    graph_safe = False
    scales_seen = 0

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.width, self.inner, self.prefix = int(params["width"]), int(params["inner"]), prefix

    def tensor_specs(self):
        return {self.prefix + "toy.w1.weight": TensorSpec((self.inner, self.width)),
                self.prefix + "toy.w2.weight": TensorSpec((self.width, self.inner))}

    def load(self, tensors):
        self.w1 = tensors[self.prefix + "toy.w1.weight"].float()
        self.w2 = tensors[self.prefix + "toy.w2.weight"].float()

    def takes_row_scale(self):
        return True

    def forward(self, x, residual, ctx):
        xf = x.float()
        scale = ctx.take_row_scale(x)
        if scale is not None:
            type(self).scales_seen += 1
            xf = xf * scale.values()[:x.shape[0], None]
        return residual + torch.tanh(xf @ self.w1.t()) @ self.w2.t()


def test_toy_feed_forward_that_takes_row_scales(tmp_path):
    from braidinfer_b200.engine import Engine
    from braidinfer_b200.models import architecture_for
    from tiny import TINY_A, random_prompts
    import plain_mistral as P
    FEED_FORWARDS.register("toy_scale_aware", ScaleAwarePerceptron)
    try:
        arch = architecture_for(TINY_A)
        cfg = arch.config_from_dict(TINY_A)
        base = arch.build_spec(cfg)
        layers = tuple(dataclasses.replace(ls, feed_forward=PartSpec("toy_scale_aware", {"width": cfg.hidden_size, "inner": 48}))
                       for ls in base.layers)
        spec = dataclasses.replace(base, layers=layers)
        eng = Engine.from_spec(spec, 4, dtype="bfloat16", max_tokens=512, max_slots=2, verbose=False)
        w = {n_: t.double() for n_, t in eng.drawn.items()}

        pcfg = P.PlainConfig(TINY_A)

        def plain(tokens):
            pos = torch.arange(len(tokens))
            h = P.embedding(w["model.embed_tokens.weight"], tokens, torch.float64)
            for layer in range(cfg.num_hidden_layers):
                pre = f"model.layers.{layer}."
                h = h + P.attention_block(h, w, pre, pcfg, layer, pos)
                n = P.rmsnorm(h, w[pre + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
                h = h + torch.tanh(n @ w[pre + "toy.w1.weight"].t()) @ w[pre + "toy.w2.weight"].t()
            return P.linear(P.rmsnorm(h, w["model.norm.weight"], cfg.rms_norm_eps), w["lm_head.weight"])

        toks = random_prompts(cfg.vocab_size, [40], seed=5)[0]
        want = plain(toks)
        s = eng.open()
        ScaleAwarePerceptron.scales_seen = 0
        got = [eng.step([(s, toks[:30])], want="last")]
        for t in toks[30:]:
            got.append(eng.step([(s, [t])], want="last"))
        got = torch.cat(got)
        assert ScaleAwarePerceptron.scales_seen >= 2 * 11          # every feed-forward call of the steps of few tokens
        assert (got.double().cpu() - want[29:]).abs().max() < 1.5e-2
        eng.check()
    finally:
        FEED_FORWARDS.unregister("toy_scale_aware")


# ---------------------------------------------------------------------------------------------
# The parts nobody had swapped yet, each written to the interface that braidinfer_b200/parts/base.py
# documents and registered from here: a norm with a mean and a bias (also as the model's final norm,
# where it is handed the wanted rows only), a block that runs mixer and feed-forward side by side
# from one norm, an embedding with a scale, a head that caps its logits, and attention without any
# position encoding (the built-in "none").
from braidinfer_b200.parts import BLOCKS, EMBEDDINGS, HEADS, NORMS, Block, Embedding, Head, Norm


class ToyLayerNorm(Norm):
    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.width, self.eps = int(params["width"]), float(params["eps"])
        self.wn, self.bn = prefix + params["name"] + ".weight", prefix + params["name"] + ".bias"

    def tensor_specs(self):
        return {self.wn: TensorSpec((self.width,), init="one_plus_normal"), self.bn: TensorSpec((self.width,))}

    def load(self, tensors):
        self.w, self.b = tensors[self.wn].float(), tensors[self.bn].float()

    def forward(self, x, ctx, row_index=None, rows=None):
        if row_index is not None:                       # the final norm: the wanted rows only
            x = x[row_index[:rows].long()]
        mu = x.mean(-1, keepdim=True)
        var = ((x - mu) ** 2).mean(-1, keepdim=True)
        return ((x - mu) * torch.rsqrt(var + self.eps) * self.w + self.b).to(self.rt.act_dtype)


class SideBySideBlock(Block):
    """h + mixer(norm(h)) + feed_forward(norm(h)): one norm feeds both."""

    def forward(self, h, ctx, cache, state):
        ctx.resolve(h)                                  # the norm here knows nothing of deferred sums
        x = self.mixer_norm.forward(h, ctx)
        h = self.mixer.forward(x, h, ctx, cache, state)
        ctx.resolve(h)
        return self.feed_forward.forward(x, h, ctx)


class ScaledEmbedding(Embedding):
    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.vocab, self.width, self.scale = int(params["vocab_size"]), int(params["hidden_size"]), float(params["scale"])
        self.name = prefix + "model.embed_tokens.weight"

    def tensor_specs(self):
        return {self.name: TensorSpec((self.vocab, self.width))}

    def load(self, tensors):
        self.weight = tensors[self.name]

    def forward(self, token_ids, rows):
        return self.weight[token_ids[:rows].long()].float() * self.scale


class CappedHead(Head):
    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.vocab, self.width, self.cap = int(params["vocab_size"]), int(params["hidden_size"]), float(params["cap"])
        self.name = prefix + "lm_head.weight"

    def tensor_specs(self):
        return {self.name: TensorSpec((self.vocab, self.width))}

    def load(self, tensors):
        self.w = tensors[self.name].float()

    def forward(self, x):
        return self.cap * torch.tanh(x.float() @ self.w.t() / self.cap)


def plain_toy_model_3(weights, cfg, tokens, scale, cap, eps):
    import plain_mistral as P
    w = {k: v.double() for k, v in weights.items()}
    T = len(tokens)
    nqh, nkh, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim

    def layer_norm(x, name):
        mu = x.mean(-1, keepdim=True)
        var = ((x - mu) ** 2).mean(-1, keepdim=True)
        return (x - mu) * torch.rsqrt(var + eps) * w[name + ".weight"] + w[name + ".bias"]

    h = P.embedding(w["model.embed_tokens.weight"], tokens, torch.float64) * scale
    for layer in range(cfg.num_hidden_layers):
        pre = f"model.layers.{layer}."
        n = layer_norm(h, pre + "toy_norm")
        q = P.linear(n, w[pre + "self_attn.q_proj.weight"]).view(T, nqh, hd)          # no position encoding at all
        k = P.linear(n, w[pre + "self_attn.k_proj.weight"]).view(T, nkh, hd)
        v = P.linear(n, w[pre + "self_attn.v_proj.weight"]).view(T, nkh, hd)
        a = P.linear(P.attention(q, k, v, cfg.layer_window(layer)).reshape(T, nqh * hd), w[pre + "self_attn.o_proj.weight"])
        f = P.swiglu(n, w[pre + "mlp.gate_proj.weight"], w[pre + "mlp.up_proj.weight"], w[pre + "mlp.down_proj.weight"])
        h = h + a + f
    h = layer_norm(h, "toy_final")
    return cap * torch.tanh(P.linear(h, w["lm_head.weight"]) / cap)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_norm_block_embedding_head_and_no_position_encoding(dtype):
    from braidinfer_b200.engine import Engine
    from braidinfer_b200.models import architecture_for
    from tiny import TINY_B, random_prompts
    NORMS.register("toy_layer_norm", ToyLayerNorm)
    BLOCKS.register("toy_side_by_side", SideBySideBlock)
    EMBEDDINGS.register("toy_scaled_embedding", ScaledEmbedding)
    HEADS.register("toy_capped_head", CappedHead)
    try:
        arch = architecture_for(TINY_B)
        cfg = arch.config_from_dict(TINY_B)
        base = arch.build_spec(cfg)
        eps, scale, cap = 1e-4, 3.0, 0.4
        layers = []
        for ls in base.layers:
            mp = dict(ls.mixer.params)
            mp["position_encoding"] = PartSpec("none", {"head_dim": cfg.head_dim})
            layers.append(dataclasses.replace(
                ls, block="toy_side_by_side", mixer=PartSpec("gqa_attention", mp),
                mixer_norm=PartSpec("toy_layer_norm", {"width": cfg.hidden_size, "eps": eps, "name": "toy_norm"}),
                feed_forward_norm=PartSpec("toy_layer_norm", {"width": cfg.hidden_size, "eps": eps, "name": "toy_norm"})))
        spec = dataclasses.replace(
            base, layers=tuple(layers),
            embedding=PartSpec("toy_scaled_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                                        "scale": scale}),
            final_norm=PartSpec("toy_layer_norm", {"width": cfg.hidden_size, "eps": eps, "name": "toy_final"}),
            head=PartSpec("toy_capped_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "cap": cap}))
        eng = Engine.from_spec(spec, 13, dtype=dtype, max_tokens=512, max_slots=3, verbose=False,
                               scale={"toy_norm.bias": 10.0, "toy_final.bias": 10.0, "lm_head.weight": 10.0})
        names = set(eng.model.tensor_specs())
        assert {"model.layers.2.toy_norm.bias", "toy_final.weight", "lm_head.weight"} <= names
        assert not any("layernorm" in n or n == "model.norm.weight" for n in names)
        assert eng.use_graphs                     # every part here can be replayed by a graph
        w64 = {n_: t.double() for n_, t in eng.drawn.items()}
        prompts = random_prompts(cfg.vocab_size, [70, 9, 21], seed=3)
        want = [plain_toy_model_3(w64, cfg, p, scale, cap, eps) for p in prompts]
        assert max(w_.abs().max().item() for w_ in want) > 0.9 * cap          # the cap does bite
        tol = 2e-5 if dtype == "float32" else 1.5e-2
        slots = [eng.open() for _ in prompts]
        cut = [64, 3, 12]
        got = eng.step([(s, p[:c]) for s, p, c in zip(slots, prompts, cut)], want=[[0, 63], [2], list(range(12))])
        assert (got[0].double().cpu() - want[0][0]).abs().max() < tol         # wanted rows, gathered by the final norm
        assert (got[1].double().cpu() - want[0][63]).abs().max() < tol
        assert (got[2].double().cpu() - want[1][2]).abs().max() < tol
        assert (got[3:].double().cpu() - want[2][:12]).abs().max() < tol
        for t in range(6):                                                    # the later ones through a CUDA graph
            out = eng.step([(slots[i], [prompts[i][cut[i] + t]]) for i in range(3)], want="last")
            for i in range(3):
                assert (out[i].double().cpu() - want[i][cut[i] + t]).abs().max() < tol
        assert eng.graph_replays >= 4
        eng.check()
        # generation through the entry point works for a model that no configuration describes
        import braidinfer_b200 as lib
        m = lib.Model(eng, max_batch=3)
        for s in slots:
            eng.close(s)
        outs = m.generate([p[:5] for p in prompts], None, None, 4)
        assert [len(o.tokens) for o in outs] == [4, 4, 4] and m.config is None
    finally:
        NORMS.unregister("toy_layer_norm")
        BLOCKS.unregister("toy_side_by_side")
        EMBEDDINGS.unregister("toy_scaled_embedding")
        HEADS.unregister("toy_capped_head")


# ---------------------------------------------------------------------------------------------
# A whole toy architecture, defined and registered here only: its own config.json keys, its own
# typed configuration, its own recipe of parts (the running-mean mixer above in layer 0, attention
# in layer 1).  The library's files stay as they are: the random-weights writer, the loader, the
# cache, the step function, the generation loop and the trace replay all find it through the
# registry, by the name in config.json.
@dataclasses.dataclass(frozen=True)
class ToyConfig:
    width: int
    heads: int
    groups: int
    head_size: int
    inner: int
    words: int
    wavelength: float
    eps: float
    longest: int
    end_word: int

    @classmethod
    def from_dict(cls, d):
        return cls(int(d["width"]), int(d["heads"]), int(d["groups"]), int(d["head_size"]), int(d["inner"]),
                   int(d["words"]), float(d["wavelength"]), float(d["eps"]), int(d["longest"]), int(d["end_word"]))


def build_toy_spec(c: ToyConfig):
    from braidinfer_b200.parts.spec import ModelSpec, ScheduleEntry

    def norm(name):
        return PartSpec("rmsnorm", {"width": c.width, "eps": c.eps, "name": name})

    rope = PartSpec("rope", {"head_dim": c.head_size, "theta": c.wavelength, "rope_dim": c.head_size, "pairing": "half"})
    mixers = [PartSpec("toy_running_mean", {"width": c.width}),
              PartSpec("gqa_attention", {"hidden_size": c.width, "num_heads": c.heads, "num_kv_heads": c.groups,
                                         "head_dim": c.head_size, "window": 0, "position_encoding": rope})]
    layers = tuple(LayerSpec(block="prenorm_residual", prefix=f"model.layers.{i}.", mixer=m,
                             mixer_norm=norm("input_layernorm.weight"),
                             feed_forward=PartSpec("swiglu", {"hidden_size": c.width, "intermediate_size": c.inner}),
                             feed_forward_norm=norm("post_attention_layernorm.weight"))
                   for i, m in enumerate(mixers))
    return ModelSpec(hidden_size=c.width, vocab_size=c.words,
                     embedding=PartSpec("token_embedding", {"vocab_size": c.words, "hidden_size": c.width,
                                                            "name": "model.embed_tokens.weight"}),
                     layers=layers, schedule=(ScheduleEntry(0), ScheduleEntry(1)), final_norm=norm("model.norm.weight"),
                     head=PartSpec("linear_head", {"vocab_size": c.words, "hidden_size": c.width,
                                                   "name": "lm_head.weight", "tied": False}),
                     max_position=c.longest, eos_token_ids=(c.end_word,), bos_token_id=None)


TOY_CONFIG_JSON = {"architectures": ["ToyRunningMeanLM"], "width": 64, "heads": 4, "groups": 2, "head_size": 16,
                   "inner": 176, "words": 256, "wavelength": 10000.0, "eps": 1e-5, "longest": 512, "end_word": 2}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_from_config_json_to_generation_and_replay(dtype, tmp_path):
    import json
    import numpy as np
    import braidinfer_b200 as lib
    from braidinfer_b200.config.errors import UnknownArchitectureError
    from braidinfer_b200.models import architecture_for
    from braidinfer_b200.models.registry import ARCHITECTURES, Architecture, register_architecture
    from braidinfer_b200.weights import write_random_model
    from tiny import TINY_A, random_prompts, read_weights
    folder = str(tmp_path / "toy")
    with pytest.raises(UnknownArchitectureError):
        write_random_model(TOY_CONFIG_JSON, folder, 3)
    MIXERS.register("toy_running_mean", RunningMeanMixer)
    register_architecture(Architecture("ToyRunningMeanLM", ToyConfig.from_dict, build_toy_spec))
    try:
        write_random_model(TOY_CONFIG_JSON, folder, 3)
        model = lib.load(folder, dtype=dtype, max_seq_len=128, max_batch=3, verbose=False)
        assert isinstance(model.config, ToyConfig) and model.engine.use_graphs is False
        # the oracle: the same arithmetic, whole sequences, float64; its layer 1 is the plain Mistral layer
        # at the sizes the toy keys give
        plain_cfg = architecture_for(TINY_A).config_from_dict(TINY_A)
        assert (plain_cfg.hidden_size, plain_cfg.num_attention_heads, plain_cfg.num_key_value_heads, plain_cfg.head_dim,
                plain_cfg.intermediate_size, plain_cfg.vocab_size) == (64, 4, 2, 16, 176, 256)
        w64 = {n: t.double() for n, t in read_weights(folder).items()}
        tol = 2e-5 if dtype == "float32" else 1.5e-2

        def plain(tokens):
            return plain_running_mean_model(w64, plain_cfg, list(tokens), TOY_CONFIG_JSON["eps"])

        # trace replay: two requests of unequal length start together, go on token by token, the shorter ends first
        prompts = random_prompts(256, [11, 5], seed=4)
        lines = [{"step": 0, "entries": [{"id": "a", "tokens": prompts[0][:8], "want": [0, 7]},
                                         {"id": "b", "tokens": prompts[1][:3], "want": [2]}], "end": []},
                 {"step": 1, "entries": [{"id": "a", "tokens": [prompts[0][8]], "want": [0]},
                                         {"id": "b", "tokens": [prompts[1][3]], "want": [0]}], "end": []},
                 {"step": 2, "entries": [{"id": "a", "tokens": [prompts[0][9]], "want": [0]},
                                         {"id": "b", "tokens": [prompts[1][4]], "want": [0]}], "end": ["b"]},
                 {"step": 3, "entries": [{"id": "a", "tokens": [prompts[0][10]], "want": [0]}], "end": ["a"]}]
        out = str(tmp_path / "out")
        assert model.replay(lines, out) == len(lines)
        wa, wb = plain(prompts[0]), plain(prompts[1])
        want = {0: [wa[0], wa[7], wb[2]], 1: [wa[8], wb[3]], 2: [wa[9], wb[4]], 3: [wa[10]]}
        for step, rows in want.items():
            got = torch.from_numpy(np.fromfile(f"{out}/{step}.f32", dtype="<f4").reshape(len(rows), 256))
            assert (got.double() - torch.stack(rows)).abs().max() < tol
        assert model.engine.cache.pages_in_use() == [0]
        # greedy generation through the entry point: token by token the plain model's argmax, and the toy's own
        # end word stops a sequence
        starts = random_prompts(256, [6, 3, 9], seed=5)
        outs = model.generate(starts, lib.SamplingParams.greedy(), max_new_tokens=5)
        for start, o in zip(starts, outs):
            seq = list(start)
            for tok in o.tokens:
                lg = plain(seq)[-1]
                top2 = torch.topk(lg, 2).values
                if (top2[0] - top2[1]).item() > 4 * tol:          # a near tie may fall either way in bfloat16
                    assert tok == int(lg.argmax())
                seq.append(tok)
            assert TOY_CONFIG_JSON["end_word"] not in o.tokens
            assert o.finish_reason in ("stop", "length") and (o.finish_reason == "stop" or len(o.tokens) == 5)
        model.engine.check()
    finally:
        ARCHITECTURES.pop("ToyRunningMeanLM", None)
        MIXERS.unregister("toy_running_mean")
