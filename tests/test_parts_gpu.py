"""Each part alone against the plain implementation, a schedule that names a layer
twice and lets a layer read another's cache, and a toy mixer with state of its
own that is registered, built and stepped from this file alone."""

from __future__ import annotations

import math

import pytest
import torch

import helpers
import plain_qwen3

pytestmark = pytest.mark.gpu


def env(hidden, dtype=torch.float32, prefix="p"):
    from vllm_from_scratch_b200.parts import PartEnv
    return PartEnv(hidden, dtype, torch.device("cuda"), prefix)


def test_rms_norm_part():
    from vllm_from_scratch_b200.parts import NORMS
    norm = NORMS.get("rms_norm")({"eps": 1e-5}, env(96))
    assert norm.expected_weights()["weight"].shape == (96,)
    weight = torch.rand(96, device="cuda") + 0.5
    norm.load_weights({"weight": weight})
    x = torch.randn(7, 96, device="cuda")
    residual = torch.randn(7, 96, device="cuda")
    expected_sum = residual + x
    out = norm.forward(x, residual)
    assert torch.allclose(residual, expected_sum, atol=1e-6)
    assert torch.allclose(out, plain_qwen3.rms_norm(expected_sum, weight, 1e-5), atol=1e-5)


def test_position_parts():
    from vllm_from_scratch_b200.parts import POSITION_ENCODINGS
    rotary = POSITION_ENCODINGS.get("rotary")({"theta": 1e6, "rotary_dim": 32}, env(64))
    expected = 1.0 / (1e6 ** (torch.arange(0, 32, 2, dtype=torch.float32) / 32))
    assert torch.equal(rotary.inverse_frequencies().cpu(), expected) and rotary.rotary_dim == 32
    scaled = POSITION_ENCODINGS.get("rotary")({"theta": 1e6, "rotary_dim": 32, "scaling_factor": 4.0}, env(64))
    assert torch.allclose(scaled.inverse_frequencies().cpu(), expected / 4)
    none = POSITION_ENCODINGS.get("none")({}, env(64))
    assert none.rotary_dim == 0 and none.inverse_frequencies() is None


def test_feed_forward_part():
    from vllm_from_scratch_b200.parts import FEED_FORWARDS
    part = FEED_FORWARDS.get("gated_silu")({"intermediate_size": 160}, env(96))
    shapes = {k: v.shape for k, v in part.expected_weights().items()}
    assert shapes == {"gate_proj.weight": (160, 96), "up_proj.weight": (160, 96), "down_proj.weight": (96, 160)}
    w = {name: torch.randn(*shape, device="cuda") * 0.1 for name, shape in shapes.items()}
    part.load_weights(w)
    x = torch.randn(9, 96, device="cuda")
    expected = plain_qwen3.feed_forward(x, {"m." + k: v for k, v in w.items()}, "m.")
    assert torch.allclose(part.forward(x, None), expected, atol=2e-5)


def attention_case(nq, nkv, d, hidden, window, with_norm, rotary=True):
    """An attention part with weights, and the same weights under plain names."""
    from vllm_from_scratch_b200.parts import MIXERS, POSITION_ENCODINGS
    position = (POSITION_ENCODINGS.get("rotary")({"theta": 1e4, "rotary_dim": d}, env(hidden)) if rotary
                else POSITION_ENCODINGS.get("none")({}, env(hidden)))
    part = MIXERS.get("paged_attention")(
        {"num_heads": nq, "num_kv_heads": nkv, "head_dim": d, "window": window,
         "qk_norm_eps": 1e-6 if with_norm else None}, env(hidden), position)
    g = torch.Generator(device="cuda").manual_seed(nq * d)
    weights = {}
    for name, info in part.expected_weights().items():
        if info.kind == "vector":
            weights[name] = 1 + 0.1 * torch.randn(*info.shape, device="cuda", generator=g)
        else:
            weights[name] = torch.randn(*info.shape, device="cuda", generator=g) * 0.15
    part.load_weights(weights)
    return part, weights


def run_part_in_portions(part, x, portions, page=8):
    """Drive an attention part directly: pages and context built by hand."""
    from vllm_from_scratch_b200.parts import CacheView, GroupContext, StepContext
    total = x.shape[0]
    pages = -(-total // page)
    order = torch.randperm(pages + 2).tolist()[:pages]
    keys = torch.zeros(pages + 2, part.num_kv_heads, page, part.head_dim, device="cuda")
    values = torch.zeros_like(keys)
    cache = CacheView("pages", 0, keys, values)
    outs, done = [], 0
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    for n in portions:
        positions = list(range(done, done + n))
        slots = [order[p // page] * page + p % page for p in positions]
        ctx = StepContext(num_tokens=n, num_requests=1, positions=i32(positions), query_start=i32([0, n]),
                          seq_lens=i32([done + n]), state_slots=i32([0]), token_request=i32([0] * n),
                          max_query_len=n, max_seq_len=done + n)
        ctx.groups[0] = GroupContext(page, i32([order]), i32(slots), pages)
        outs.append(part.forward(x[done:done + n].contiguous(), ctx, cache))
        done += n
    return torch.cat(outs)


@pytest.mark.parametrize("nq,nkv,d,hidden,window,with_norm", [
    (4, 2, 16, 64, None, True), (6, 2, 32, 96, None, True), (5, 5, 48, 80, 9, True), (3, 1, 32, 40, None, False)])
def test_attention_part_alone(nq, nkv, d, hidden, window, with_norm):
    part, weights = attention_case(nq, nkv, d, hidden, window, with_norm)
    x = torch.randn(37, hidden, device="cuda")
    cfg = {"heads": nq, "kv_heads": nkv, "head_dim": d, "eps": 1e-6, "theta": 1e4}
    plain_w = {"a." + k: v.cpu() for k, v in weights.items()}
    if not with_norm:
        plain_w["a.q_norm.weight"] = plain_w["a.k_norm.weight"] = None
        cfg["eps"] = None
    expected = plain_attention(x.cpu(), plain_w, cfg, window)
    for portions in ([37], [20, 1, 1, 2, 13], [1] * 37):
        out = run_part_in_portions(part, x, portions)
        assert float((out.cpu() - expected).abs().max()) < 3e-5, portions


def plain_attention(x, w, cfg, window, kv_override=None, return_kv=False):
    seq = x.shape[0]
    nq, nkv, d = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    q = (x @ w["a.q_proj.weight"].T).view(seq, nq, d)
    k = (x @ w["a.k_proj.weight"].T).view(seq, nkv, d)
    v = (x @ w["a.v_proj.weight"].T).view(seq, nkv, d)
    if cfg["eps"] is not None:
        q = plain_qwen3.rms_norm(q, w["a.q_norm.weight"], cfg["eps"])
        k = plain_qwen3.rms_norm(k, w["a.k_norm.weight"], cfg["eps"])
    cos, sin = plain_qwen3.rope_cos_sin(torch.arange(seq), d, cfg["theta"], x.dtype)
    q, k = plain_qwen3.apply_rope(q, cos, sin), plain_qwen3.apply_rope(k, cos, sin)
    if kv_override is not None:
        k, v = kv_override
    out = plain_qwen3.causal_attention(q, k, v, 1.0 / math.sqrt(d), window) @ w["a.o_proj.weight"].T
    return (out, (k, v)) if return_kv else out


# ----------------------------------------------------------- schedules as data
def small_spec(schedule, layers=2, hidden=64, vocab=97):
    from vllm_from_scratch_b200 import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    norm = {"eps": 1e-6}
    specs = [LayerSpec(
        name=f"model.layers.{i}", block=PartSpec("pre_norm"),
        mixer=PartSpec("paged_attention", {"num_heads": 4, "num_kv_heads": 2, "head_dim": 16,
                                           "window": None, "qk_norm_eps": 1e-6}, name="self_attn"),
        feed_forward=PartSpec("gated_silu", {"intermediate_size": 72}, name="mlp"),
        position=PartSpec("rotary", {"theta": 1e4, "rotary_dim": 16}),
        norms={"mixer": PartSpec("rms_norm", norm, name="input_layernorm"),
               "feed_forward": PartSpec("rms_norm", norm, name="post_attention_layernorm")}) for i in range(layers)]
    return ModelSpec(hidden_size=hidden, vocab_size=vocab, embedding=PartSpec("token_embedding", name="model.embed_tokens"),
                     layers=tuple(specs), schedule=tuple(ScheduleEntry(*entry) for entry in schedule),
                     final_norm=PartSpec("rms_norm", norm, name="model.norm"),
                     output_head=PartSpec("linear_head", {"tied": True}, name="lm_head"))


def random_weights_for(model, seed=0):
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, info in model.expected_weights().items():
        if info.kind == "vector":
            out[name] = 1 + 0.1 * torch.randn(*info.shape, generator=g)
        else:
            out[name] = torch.randn(*info.shape, generator=g) * 0.1
    return out


def plain_scheduled_logits(weights, schedule, tokens, hidden=64):
    """The plain model run in the order of ``schedule``; an entry with cache_from
    attends over the keys and values of that earlier entry."""
    cfg = {"heads": 4, "kv_heads": 2, "head_dim": 16, "eps": 1e-6, "theta": 1e4}
    h = weights["model.embed_tokens.weight"][torch.tensor(tokens)]
    kept = {}
    for index, (layer, source) in enumerate(schedule):
        prefix = f"model.layers.{layer}."
        w = {"a." + k[len(prefix + "self_attn."):]: v for k, v in weights.items() if k.startswith(prefix + "self_attn.")}
        normed = plain_qwen3.rms_norm(h, weights[prefix + "input_layernorm.weight"], 1e-6)
        out, kv = plain_attention(normed, w, cfg, None, kv_override=kept.get(source), return_kv=True)
        if source is None:
            kept[index] = kv
        h = h + out
        normed = plain_qwen3.rms_norm(h, weights[prefix + "post_attention_layernorm.weight"], 1e-6)
        h = h + plain_qwen3.feed_forward(normed, weights, prefix + "mlp.")
    return plain_qwen3.rms_norm(h, weights["model.norm.weight"], 1e-6) @ weights["model.embed_tokens.weight"].T


def test_schedule_names_a_layer_twice_and_shares_a_cache():
    from vllm_from_scratch_b200 import ModelRunner
    from vllm_from_scratch_b200.parts import DecoderModel
    schedule = [(0, None), (1, None), (0, None), (1, 1)]
    spec = small_spec(schedule)
    weights = random_weights_for(DecoderModel(spec, torch.float32, "cpu"))
    runner = ModelRunner(spec, weights, "float32", 8, 24, 2, device="cuda")
    # three executions own a cache, the fourth reads the second one's
    assert len(runner.storage.groups) == 1 and runner.storage.groups[0].entries == [0, 1, 2]
    assert runner.storage.views[3].writable is False
    assert runner.storage.views[3].keys.data_ptr() == runner.storage.views[1].keys.data_ptr()
    tokens = helpers.random_tokens(97, 50, seed=4)
    expected = plain_scheduled_logits(weights, schedule, tokens)
    for steps in ([[("r", 50)]], [[("r", 17)], [("r", 2)], [("r", 30)], [("r", 1)]]):
        result = helpers.run_schedule(runner, {"r": tokens}, steps)["r"]
        assert float((result - expected).abs().max()) < 3e-5


# ------------------------------------------------------- a toy mixer with state
def test_toy_mixer_with_state_registers_builds_and_steps():
    """A mixer defined here, with one float32 vector of state per request: y_t =
    s_t W, s_t = decay * s_{t-1} + x_t.  It is registered from the test, placed in
    a model beside an attention layer, and stepped in portions, mixed with another
    request, and again after its slot was used by someone else."""
    from vllm_from_scratch_b200 import LayerSpec, ModelRunner, PartSpec
    from vllm_from_scratch_b200.parts import MIXERS, DecoderModel, Mixer, StateNeed, WeightInfo
    import dataclasses

    class RunningSumMixer(Mixer):
        def __init__(self, params, env, position):
            super().__init__(params, env, position)
            self.decay = float(params["decay"])
            self.weight = None

        def expected_weights(self):
            return {"mix.weight": WeightInfo((self.env.hidden_size, self.env.hidden_size))}

        def load_weights(self, tensors):
            self.weight = tensors["mix.weight"]

        def cache_need(self):
            return StateNeed((self.env.hidden_size,), torch.float32)

        def forward(self, x, ctx, cache):
            assert cache.kind == "state"
            out = torch.empty_like(x)
            starts = ctx.host_query_start
            for row, slot in enumerate(ctx.host_state_slots):
                state = cache.state[slot]
                for t in range(starts[row], starts[row + 1]):
                    state = self.decay * state + x[t].float()
                    out[t] = (state @ self.weight.float().T).to(x.dtype)
                cache.state[slot] = state
            return out

    MIXERS.register("toy_running_sum")(RunningSumMixer)
    try:
        base = small_spec([(0, None), (1, None)])
        toy_layer = dataclasses.replace(base.layers[1], mixer=PartSpec("toy_running_sum", {"decay": 0.7}, name="toy"),
                                        position=PartSpec("none"))
        spec = dataclasses.replace(base, layers=(base.layers[0], toy_layer))
        weights = random_weights_for(DecoderModel(spec, torch.float32, "cpu"), seed=3)
        assert "model.layers.1.toy.mix.weight" in weights
        runner = ModelRunner(spec, weights, "float32", 8, 32, 2, device="cuda")
        assert runner.storage.has_state and not runner.manager.prefix_caching

        def plain(tokens):
            cfg = {"heads": 4, "kv_heads": 2, "head_dim": 16, "eps": 1e-6, "theta": 1e4}
            h = weights["model.embed_tokens.weight"][torch.tensor(tokens)]
            p = "model.layers.0."
            w = {"a." + k[len(p + "self_attn."):]: v for k, v in weights.items() if k.startswith(p + "self_attn.")}
            h = h + plain_attention(plain_qwen3.rms_norm(h, weights[p + "input_layernorm.weight"], 1e-6), w, cfg, None)
            h = h + plain_qwen3.feed_forward(plain_qwen3.rms_norm(h, weights[p + "post_attention_layernorm.weight"], 1e-6), weights, p + "mlp.")
            p = "model.layers.1."
            normed = plain_qwen3.rms_norm(h, weights[p + "input_layernorm.weight"], 1e-6)
            state = torch.zeros(64)
            mixed = []
            for t in range(len(tokens)):
                state = 0.7 * state + normed[t]
                mixed.append(state @ weights[p + "toy.mix.weight"].T)
            h = h + torch.stack(mixed)
            h = h + plain_qwen3.feed_forward(plain_qwen3.rms_norm(h, weights[p + "post_attention_layernorm.weight"], 1e-6), weights, p + "mlp.")
            return plain_qwen3.rms_norm(h, weights["model.norm.weight"], 1e-6) @ weights["model.embed_tokens.weight"].T

        sequences = {rid: helpers.random_tokens(97, n, seed=n) for rid, n in {"a": 40, "b": 23, "c": 31}.items()}
        expected = {rid: plain(toks) for rid, toks in sequences.items()}
        # a and b share steps; c comes later and gets a slot that was used before
        steps = [[("a", 9)], [("a", 1), ("b", 5)], [("b", 18), ("a", 2)], [("a", 28)], [("c", 30)], [("c", 1)]]
        results = helpers.run_schedule(runner, sequences, steps)
        for rid in sequences:
            assert float((results[rid] - expected[rid]).abs().max()) < 5e-5, rid
    finally:
        MIXERS.unregister("toy_running_sum")


# ------------------------------------- a toy feed-forward with routing, a toy position encoding
def test_toy_routed_feed_forward_and_toy_frequencies_register_build_and_step():
    """Two more parts defined here and registered from the test: a feed-forward that sends
    each token to one of three small experts (router logits and the choice in float32), and
    a position encoding of the rotary family with frequencies of its own over half of the
    head.  Layer 0 keeps the model's parts, layer 1 takes both toys; the model is stepped
    whole, in portions and mixed with another request."""
    from vllm_from_scratch_b200 import ModelRunner, PartSpec
    from vllm_from_scratch_b200.parts import (FEED_FORWARDS, POSITION_ENCODINGS, DecoderModel, FeedForward,
                                              PositionEncoding, WeightInfo)
    import dataclasses

    class TopOneExperts(FeedForward):
        def __init__(self, params, env):
            super().__init__(params, env)
            self.experts = int(params["experts"])
            self.router = self.w = None

        def expected_weights(self):
            h = self.env.hidden_size
            return {"router.weight": WeightInfo((self.experts, h)), "experts.weight": WeightInfo((self.experts * h, h))}

        def load_weights(self, tensors):
            self.router, self.w = tensors["router.weight"], tensors["experts.weight"]

        def forward(self, x, ctx):
            h = self.env.hidden_size
            logits = x.float() @ self.router.float().T                  # float32 router
            choice = logits.argmax(dim=-1)
            gate = torch.softmax(logits, dim=-1).gather(1, choice[:, None])
            w = self.w.float().view(self.experts, h, h)[choice]         # [T, h, h]
            return (gate * torch.einsum("tk,tnk->tn", x.float(), w)).to(x.dtype)

    class BandFrequencies(PositionEncoding):
        def __init__(self, params, env):
            super().__init__(params, env)
            self.rotary_dim = int(params["rotary_dim"])
            self._inv = torch.tensor(params["inverse_frequencies"], dtype=torch.float32, device=env.device)
            assert self._inv.numel() == self.rotary_dim // 2

        def inverse_frequencies(self):
            return self._inv

    band = [1.0, 0.5, 0.03, 0.002]                                      # 8 of the 16 channels of a head rotate
    FEED_FORWARDS.register("toy_top_one_experts")(TopOneExperts)
    POSITION_ENCODINGS.register("toy_band_frequencies")(BandFrequencies)
    try:
        base = small_spec([(0, None), (1, None)])
        toy = dataclasses.replace(
            base.layers[1], feed_forward=PartSpec("toy_top_one_experts", {"experts": 3}, name="moe"),
            position=PartSpec("toy_band_frequencies", {"rotary_dim": 8, "inverse_frequencies": band}))
        spec = dataclasses.replace(base, layers=(base.layers[0], toy))
        weights = random_weights_for(DecoderModel(spec, torch.float32, "cpu"), seed=8)
        assert "model.layers.1.moe.router.weight" in weights and "model.layers.1.mlp.down_proj.weight" not in weights
        runner = ModelRunner(spec, weights, "float32", 8, 32, 2, device="cuda")

        def plain(tokens):
            cfg = {"heads": 4, "kv_heads": 2, "head_dim": 16, "eps": 1e-6, "theta": 1e4}
            h = weights["model.embed_tokens.weight"][torch.tensor(tokens)]
            p = "model.layers.0."
            w = {"a." + k[len(p + "self_attn."):]: v for k, v in weights.items() if k.startswith(p + "self_attn.")}
            h = h + plain_attention(plain_qwen3.rms_norm(h, weights[p + "input_layernorm.weight"], 1e-6), w, cfg, None)
            h = h + plain_qwen3.feed_forward(plain_qwen3.rms_norm(h, weights[p + "post_attention_layernorm.weight"], 1e-6), weights, p + "mlp.")
            p = "model.layers.1."
            x = plain_qwen3.rms_norm(h, weights[p + "input_layernorm.weight"], 1e-6)
            seq = len(tokens)
            q = plain_qwen3.rms_norm((x @ weights[p + "self_attn.q_proj.weight"].T).view(seq, 4, 16), weights[p + "self_attn.q_norm.weight"], 1e-6)
            k = plain_qwen3.rms_norm((x @ weights[p + "self_attn.k_proj.weight"].T).view(seq, 2, 16), weights[p + "self_attn.k_norm.weight"], 1e-6)
            v = (x @ weights[p + "self_attn.v_proj.weight"].T).view(seq, 2, 16)
            angles = torch.arange(seq, dtype=torch.float32)[:, None] * torch.tensor(band)[None, :]
            q, k = plain_qwen3.apply_rope(q, angles.cos(), angles.sin()), plain_qwen3.apply_rope(k, angles.cos(), angles.sin())
            h = h + plain_qwen3.causal_attention(q, k, v, 0.25, None) @ weights[p + "self_attn.o_proj.weight"].T
            x = plain_qwen3.rms_norm(h, weights[p + "post_attention_layernorm.weight"], 1e-6)
            logits = x @ weights[p + "moe.router.weight"].T
            choice = logits.argmax(dim=-1)
            gate = torch.softmax(logits, dim=-1).gather(1, choice[:, None])
            experts = weights[p + "moe.experts.weight"].view(3, 64, 64)[choice]
            h = h + gate * torch.einsum("tk,tnk->tn", x, experts)
            return plain_qwen3.rms_norm(h, weights["model.norm.weight"], 1e-6) @ weights["model.embed_tokens.weight"].T

        sequences = {rid: helpers.random_tokens(97, n, seed=3 * n) for rid, n in {"a": 45, "b": 19}.items()}
        expected = {rid: plain(toks) for rid, toks in sequences.items()}
        for steps in ([[("a", 45), ("b", 19)]], [[("a", 7)], [("a", 2), ("b", 11)], [("b", 8), ("a", 30)], [("a", 6)]]):
            results = helpers.run_schedule(runner, sequences, steps)
            for rid in sequences:
                assert float((results[rid] - expected[rid]).abs().max()) < 5e-5, rid
    finally:
        FEED_FORWARDS.unregister("toy_top_one_experts")
        POSITION_ENCODINGS.unregister("toy_band_frequencies")


# ---------------------------------------------- what the engine does with parts it does not know
def _plain_attention_layer(weights, h, layer, cfg):
    p = f"model.layers.{layer}."
    w = {"a." + k[len(p + "self_attn."):]: v for k, v in weights.items() if k.startswith(p + "self_attn.")}
    h = h + plain_attention(plain_qwen3.rms_norm(h, weights[p + "input_layernorm.weight"], 1e-6), w, cfg, None)
    return h + plain_qwen3.feed_forward(
        plain_qwen3.rms_norm(h, weights[p + "post_attention_layernorm.weight"], 1e-6), weights, p + "mlp.")


def _greedy_by(plain, prompt, new_tokens):
    tokens, margins = list(prompt), []
    for _ in range(new_tokens):
        logits = plain(tokens)[-1]
        top = torch.topk(logits, 2).values
        margins.append(float(top[0] - top[1]))
        tokens.append(int(logits.argmax()))
    return tokens[len(prompt):], margins


@pytest.mark.parametrize("device_path", [False, True])
def test_state_mixer_through_the_engine_with_graphs_asked_for(device_path):
    """The toy mixer with state of its own, driven by ``LLMEngine`` with graph replay asked for.
    Written with host lists (``ctx.host_state_slots``) it does not say ``graph_safe``: the engine
    must then run without graphs rather than bake one step's slots into a graph.  Written so
    that a decode step reads its slots from device data, and saying so, it is replayed.  Either
    way the greedy tokens are the plain model's."""
    import dataclasses
    import vllm_from_scratch_b200 as engine
    from vllm_from_scratch_b200 import ModelRunner, PartSpec
    from vllm_from_scratch_b200.parts import MIXERS, DecoderModel, Mixer, StateNeed, WeightInfo

    class RunningSum(Mixer):
        graph_safe = device_path

        def __init__(self, params, env, position):
            super().__init__(params, env, position)
            self.decay, self.weight = float(params["decay"]), None

        def expected_weights(self):
            return {"mix.weight": WeightInfo((self.env.hidden_size, self.env.hidden_size))}

        def load_weights(self, tensors):
            self.weight = tensors["mix.weight"]

        def cache_need(self):
            return StateNeed((self.env.hidden_size,), torch.float32)

        def forward(self, x, ctx, cache):
            if device_path and ctx.max_query_len == 1 and x.shape[0] == ctx.num_requests:
                # one token per request: the slots come from the device, nothing from the host
                slots = ctx.state_slots.long()
                state = self.decay * cache.state[slots] + x.float()
                cache.state[slots] = state
                return (state @ self.weight.float().T).to(x.dtype)
            out = torch.empty_like(x)
            starts = ctx.host_query_start
            for row, slot in enumerate(ctx.host_state_slots):
                state = cache.state[slot]
                for t in range(starts[row], starts[row + 1]):
                    state = self.decay * state + x[t].float()
                    out[t] = (state @ self.weight.float().T).to(x.dtype)
                cache.state[slot] = state
            return out

    kind = f"toy_running_sum_{int(device_path)}"
    MIXERS.register(kind)(RunningSum)
    try:
        base = small_spec([(0, None), (1, None)])
        toy_layer = dataclasses.replace(base.layers[1], mixer=PartSpec(kind, {"decay": 0.6}, name="toy"),
                                        position=PartSpec("none"))
        spec = dataclasses.replace(base, layers=(base.layers[0], toy_layer))
        weights = random_weights_for(DecoderModel(spec, torch.float32, "cpu"), seed=5)
        cfg = {"heads": 4, "kv_heads": 2, "head_dim": 16, "eps": 1e-6, "theta": 1e4}

        def plain(tokens):
            h = _plain_attention_layer(weights, weights["model.embed_tokens.weight"][torch.tensor(tokens)], 0, cfg)
            p = "model.layers.1."
            normed = plain_qwen3.rms_norm(h, weights[p + "input_layernorm.weight"], 1e-6)
            state, mixed = torch.zeros(64), []
            for t in range(len(tokens)):
                state = 0.6 * state + normed[t]
                mixed.append(state @ weights[p + "toy.mix.weight"].T)
            h = h + torch.stack(mixed)
            h = h + plain_qwen3.feed_forward(plain_qwen3.rms_norm(h, weights[p + "post_attention_layernorm.weight"], 1e-6), weights, p + "mlp.")
            return plain_qwen3.rms_norm(h, weights["model.norm.weight"], 1e-6) @ weights["model.embed_tokens.weight"].T

        runner = ModelRunner(spec, weights, "float32", 8, 48, 3, device="cuda")
        llm = engine.LLMEngine(engine.EngineConfig(
            engine.ModelConfig("(toy)", "float32", 96), engine.CacheConfig(8, 48),
            engine.SchedulerConfig(3, 32)), runner=runner)
        if device_path:
            assert llm.decode_graphs is not None and llm.mixed_graphs is None and not llm.graphs_refused_by_parts
        else:
            assert llm.decode_graphs is None and llm.graphs_refused_by_parts
        # five requests for three slots: slots are used again, by requests that join while others decode
        prompts = [helpers.random_tokens(97, n, seed=40 + n) for n in (9, 20, 3, 14, 6)]
        params = engine.SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
        for index, prompt in enumerate(prompts):
            llm.add_request(f"t{index}", prompt, params)
        latest = {}
        while llm.has_unfinished_requests():
            for output in llm.step():
                latest[output.request_id] = output
        if device_path:
            assert llm.decode_graphs.replays > 5, "decode steps must have been replayed"
        for index, prompt in enumerate(prompts):
            expected, margins = _greedy_by(plain, prompt, 10)
            got = latest[f"t{index}"].token_ids
            for place, (a, b) in enumerate(zip(got, expected)):
                if a != b:
                    assert margins[place] < 1e-4, f"request {index}: token {place} is {a}, expected {b}"
                    break
    finally:
        MIXERS.unregister(kind)


def test_toy_embedding_and_output_head_register_build_and_step():
    """The two ends of the model are parts like the others: an embedding that scales its rows and
    a head that caps its logits, defined and registered here, in a model that is otherwise the
    small one.  No file of the framework changes."""
    import dataclasses
    from vllm_from_scratch_b200 import ModelRunner, PartSpec
    from vllm_from_scratch_b200.parts import EMBEDDINGS, OUTPUT_HEADS, DecoderModel, Embedding, OutputHead, WeightInfo

    class ScaledEmbedding(Embedding):
        graph_safe = True

        def __init__(self, params, env):
            super().__init__(params, env)
            self.scale, self.weight = float(params["scale"]), None

        def expected_weights(self):
            return {"weight": WeightInfo((int(self.params["vocab_size"]), self.env.hidden_size))}

        def load_weights(self, tensors):
            self.weight = tensors["weight"]

        def forward(self, token_ids, ctx, residual, error_flag):
            residual.copy_(self.weight[token_ids.long()].float() * self.scale)

        def table(self):
            return self.weight

    class CappedHead(OutputHead):
        graph_safe = True

        def __init__(self, params, env):
            super().__init__(params, env)
            self.cap, self.weight = float(params["cap"]), None

        def bind_embedding(self, embedding):
            self.weight = embedding.table()

        def forward(self, normed):
            logits = normed.float() @ self.weight.float().T
            return self.cap * torch.tanh(logits / self.cap)

    EMBEDDINGS.register("toy_scaled_embedding")(ScaledEmbedding)
    OUTPUT_HEADS.register("toy_capped_head")(CappedHead)
    try:
        base = small_spec([(0, None), (1, None)])
        spec = dataclasses.replace(
            base, embedding=PartSpec("toy_scaled_embedding", {"scale": 8.0}, name="model.embed_tokens"),
            output_head=PartSpec("toy_capped_head", {"cap": 0.5}, name="lm_head"))
        weights = random_weights_for(DecoderModel(spec, torch.float32, "cpu"), seed=6)
        assert "lm_head.weight" not in weights
        runner = ModelRunner(spec, weights, "float32", 8, 16, 2, device="cuda")
        assert runner.model.graph_safe()
        cfg = {"heads": 4, "kv_heads": 2, "head_dim": 16, "eps": 1e-6, "theta": 1e4}
        tokens = helpers.random_tokens(97, 33, seed=2)
        h = weights["model.embed_tokens.weight"][torch.tensor(tokens)] * 8.0
        for layer in (0, 1):
            h = _plain_attention_layer(weights, h, layer, cfg)
        logits = plain_qwen3.rms_norm(h, weights["model.norm.weight"], 1e-6) @ weights["model.embed_tokens.weight"].T
        expected = 0.5 * torch.tanh(logits / 0.5)
        assert float(expected.abs().max()) > 0.3, "the cap must matter"
        for steps in ([[("r", 33)]], [[("r", 5)], [("r", 27)], [("r", 1)]]):
            result = helpers.run_schedule(runner, {"r": tokens}, steps)["r"]
            assert float((result - expected).abs().max()) < 3e-5
    finally:
        EMBEDDINGS.unregister("toy_scaled_embedding")
        OUTPUT_HEADS.unregister("toy_capped_head")


def test_toy_arrangements_with_four_norms_and_without_a_feed_forward():
    """Two arrangements defined and registered here: one with a norm in front of and behind both
    the mixer and the feed-forward (four norms a layer), one with a mixer only.  The layer's spec
    brings the norms by role; a layer that brings other roles than its block arranges is refused."""
    import dataclasses
    from vllm_from_scratch_b200 import LayerSpec, ModelRunner, PartSpec
    from vllm_from_scratch_b200.parts import BLOCKS, Block, DecoderModel

    def branch_norm(norm, branch):
        # a norm of the branch itself, not of the stream: add it into an empty stream
        return norm.forward(branch, torch.zeros(branch.shape, dtype=torch.float32, device=branch.device))

    class SandwichBlock(Block):
        norm_roles = ("pre_mixer", "post_mixer", "pre_feed_forward", "post_feed_forward")
        graph_safe = True

        def forward(self, x, residual, ctx, cache):
            mixed = self.mixer.forward(self.norms["pre_mixer"].forward(x, residual), ctx, cache)
            mixed = branch_norm(self.norms["post_mixer"], mixed)
            out = self.feed_forward.forward(self.norms["pre_feed_forward"].forward(mixed, residual), ctx)
            return branch_norm(self.norms["post_feed_forward"], out)

    class MixerOnlyBlock(Block):
        norm_roles = ("mixer",)
        needs_feed_forward = False
        graph_safe = True

        def forward(self, x, residual, ctx, cache):
            return self.mixer.forward(self.norms["mixer"].forward(x, residual), ctx, cache)

    BLOCKS.register("toy_sandwich")(SandwichBlock)
    BLOCKS.register("toy_mixer_only")(MixerOnlyBlock)
    try:
        base = small_spec([(0, None), (1, None)])
        norm = {"eps": 1e-6}
        sandwich = dataclasses.replace(base.layers[0], block=PartSpec("toy_sandwich"), norms={
            role: PartSpec("rms_norm", norm, name=f"norm_{index}")
            for index, role in enumerate(SandwichBlock.norm_roles)})
        mixer_only = dataclasses.replace(base.layers[1], block=PartSpec("toy_mixer_only"), feed_forward=None,
                                         norms={"mixer": PartSpec("rms_norm", norm, name="only_norm")})
        spec = dataclasses.replace(base, layers=(sandwich, mixer_only))
        weights = random_weights_for(DecoderModel(spec, torch.float32, "cpu"), seed=9)
        assert "model.layers.0.norm_3.weight" in weights and "model.layers.1.mlp.down_proj.weight" not in weights
        with pytest.raises(ValueError, match="arranges norms"):
            DecoderModel(dataclasses.replace(base, layers=(dataclasses.replace(sandwich, norms=base.layers[0].norms),
                                                           mixer_only)), torch.float32, "cpu")
        with pytest.raises(ValueError, match="needs a feed-forward"):
            DecoderModel(dataclasses.replace(base, layers=(dataclasses.replace(base.layers[0], feed_forward=None),
                                                           mixer_only)), torch.float32, "cpu")
        runner = ModelRunner(spec, weights, "float32", 8, 16, 2, device="cuda")
        cfg = {"heads": 4, "kv_heads": 2, "head_dim": 16, "eps": 1e-6, "theta": 1e4}
        tokens = helpers.random_tokens(97, 29, seed=12)
        rms = lambda t, name: plain_qwen3.rms_norm(t, weights[name], 1e-6)
        attention_weights = lambda p: {"a." + k[len(p + "self_attn."):]: v for k, v in weights.items()
                                       if k.startswith(p + "self_attn.")}
        h = weights["model.embed_tokens.weight"][torch.tensor(tokens)]
        p = "model.layers.0."
        h = h + rms(plain_attention(rms(h, p + "norm_0.weight"), attention_weights(p), cfg, None), p + "norm_1.weight")
        h = h + rms(plain_qwen3.feed_forward(rms(h, p + "norm_2.weight"), weights, p + "mlp."), p + "norm_3.weight")
        p = "model.layers.1."
        h = h + plain_attention(rms(h, p + "only_norm.weight"), attention_weights(p), cfg, None)
        expected = rms(h, "model.norm.weight") @ weights["model.embed_tokens.weight"].T
        for steps in ([[("r", 29)]], [[("r", 11)], [("r", 2)], [("r", 15)], [("r", 1)]]):
            result = helpers.run_schedule(runner, {"r": tokens}, steps)["r"]
            assert float((result - expected).abs().max()) < 3e-5
    finally:
        BLOCKS.unregister("toy_sandwich")
        BLOCKS.unregister("toy_mixer_only")
