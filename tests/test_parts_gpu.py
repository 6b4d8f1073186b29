"""Each part alone against the plain implementation's function for it, and the
generality of the assembly: a toy mixer with state of its own, defined here, is
registered, built and stepped without touching the library; a layer runs twice
in one schedule; a layer reads another layer's cache."""
import math

import numpy as np
import pytest
import torch

import go_tinygrad_b200 as lib
import plain_llama as plain
from go_tinygrad_b200.cache import Cache, StateRequest
from go_tinygrad_b200.config import Architecture, LlamaConfig, register_architecture, unregister_architecture
from go_tinygrad_b200.engine import Model, StepEntry, step
from go_tinygrad_b200.models.llama import llama_plan
from go_tinygrad_b200.parts import (Block, FeedForward, LayerSpec, Mixer, ModelPlan, PartSpec, PositionEncoding,
                                    ResidualStream, Runtime, ScheduleEntry, StepContext, build_part,
                                    register_part, unregister_part, walk)
from go_tinygrad_b200.weights import TensorSource, WeightSpec
from conftest import TINY, assert_close, make_prompts

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda" if torch.cuda.is_available() and torch.cuda.device_count() else "cpu")


def context(rt, seq_lens, starts, slots, tokens=None):
    """A StepContext for sequences that bring `seq_lens` tokens after `starts`."""
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    n = sum(seq_lens)
    return StepContext(
        rt=rt, n_tokens=n, n_seqs=len(seq_lens),
        tokens=i32(tokens if tokens is not None else [0] * n),
        positions=i32([s + j for s, l in zip(starts, seq_lens) for j in range(l)]),
        token_seq=i32([b for b, l in enumerate(seq_lens) for _ in range(l)]),
        cu_seqlens=i32(np.concatenate([[0], np.cumsum(seq_lens)]).tolist()),
        slots=i32(slots), start_pos=i32(starts), max_q_len=max(seq_lens),
        max_kv_len=max(s + l for s, l in zip(starts, seq_lens)), is_decode=all(l == 1 for l in seq_lens))


def tensors_of(folder):
    with TensorSource(folder) as src:
        return {n: src.tensor(n) for n in src.names()}


def tol(dtype):
    return dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["A", "B"])
def test_parts_alone(model_folders, plain_models, name, dtype):
    cfg, w = plain_models[name]
    raw = tensors_of(model_folders[name])
    plan = llama_plan(LlamaConfig.from_json(TINY[name]))
    rt = Runtime(DEV, dtype)
    H, V = cfg["hidden_size"], cfg["vocab_size"]
    lens, tokens = [70, 9], make_prompts(name, [79], seed=41)[0]
    ctx = context(rt, lens, [0, 0], [1, 0], tokens)
    rng = np.random.default_rng(0)
    x_np = rng.standard_normal((79, H)).astype(np.float32)
    x_act = torch.tensor(x_np, device=DEV).to(dtype)              # an activation in the compute dtype
    x_ref = x_act.float().cpu().numpy()

    # embedding
    emb = build_part("embedding", plan.embedding); emb.load(raw, rt)
    stream = emb.forward(ctx)
    np.testing.assert_array_equal(stream.residual.cpu().numpy(), plain.embed(w["model.embed_tokens.weight"], tokens))

    # norm: the pending update is added in float32, then normalised
    layer = plan.layers[1]
    norm = build_part("norm", layer.part("mixer_norm")); norm.load(raw, rt)
    res = torch.tensor(x_np, device=DEV)
    st = ResidualStream(res.clone(), x_act.clone())
    got = norm.forward(st, ctx)
    summed = x_np + x_ref
    assert st.pending is None
    np.testing.assert_allclose(st.residual.cpu().numpy(), summed, rtol=0, atol=0)
    want = plain.rms_norm(summed, w["model.layers.1.input_layernorm.weight"], cfg["rms_norm_eps"])
    torch.testing.assert_close(got.float().cpu(), torch.tensor(want).to(dtype).float(), **tol(dtype))

    # position encoding: the angles of the step's tokens
    pos = build_part("position", layer.part("mixer").params["position"]); pos.load(raw, rt)
    table = pos.rotation(ctx).cpu().numpy()
    inv = plain.rope_inv_freq(cfg)
    positions = list(range(70)) + list(range(9))
    ang = np.array(positions, dtype=np.float64)[:, None] * inv[None, :]
    np.testing.assert_allclose(table[..., 0], np.cos(ang).astype(np.float32), rtol=0, atol=1e-7)
    np.testing.assert_allclose(table[..., 1], np.sin(ang).astype(np.float32), rtol=0, atol=1e-7)
    assert pos.rotation(ctx) is pos.rotation(ctx)                 # computed once per step

    # mixer: attention over a cache of its own, two sequences in one step
    mixer = build_part("mixer", layer.part("mixer"))
    for part in walk(mixer):                                      # the mixer and the position encoding it owns
        part.load(raw, rt)
    cache = Cache([mixer.cache_requests()], [None], max_tokens=64 * 4, max_slots=2, dtype=dtype, device=DEV)
    for _ in range(2):
        cache.open_sequence()
    cache.reserve_many([(1, 70), (0, 9)]); cache.flush_tables()
    got = mixer.forward(x_act, ctx, cache.handles[0]).float().cpu().numpy()
    want = np.concatenate([plain.attention_block(x_ref[:70], list(range(70)), "model.layers.1.", cfg, inv, w),
                           plain.attention_block(x_ref[70:], list(range(9)), "model.layers.1.", cfg, inv, w)])
    scale = np.abs(want).max()
    limit = 1e-4 if dtype == torch.float32 else 4e-2
    assert np.abs(got - want).max() <= limit * max(1.0, scale)

    # feed-forward
    ff = build_part("feed_forward", layer.part("feed_forward")); ff.load(raw, rt)
    got = ff.forward(x_act, ctx).float().cpu().numpy()
    p = "model.layers.1.mlp."
    want = plain.swiglu_mlp(x_ref, w[p + "gate_proj.weight"], w[p + "up_proj.weight"], w[p + "down_proj.weight"])
    assert np.abs(got - want).max() <= limit * max(1.0, np.abs(want).max())

    # block: the whole layer; its second update stays pending, or its product has added it already
    block = build_part("block", layer.block)                      # it builds and owns its four parts
    assert [type(c) for c in block.children()] == [type(norm), type(mixer), type(norm), type(ff)]
    assert block.cache_requests() == mixer.cache_requests()
    for part in walk(block):
        part.load(raw, rt)
    cache2 = Cache([mixer.cache_requests()], [None], max_tokens=64 * 4, max_slots=2, dtype=dtype, device=DEV)
    for _ in range(2):
        cache2.open_sequence()
    cache2.reserve_many([(1, 70), (0, 9)]); cache2.flush_tables()
    st = ResidualStream(torch.tensor(x_np, device=DEV))
    block.forward(st, context(rt, lens, [0, 0], [1, 0], tokens), cache2.handles[0])
    got = (st.residual if st.pending is None else st.residual + st.pending.float()).cpu().numpy()
    want = np.concatenate([plain.decoder_layer(x_np[:70], list(range(70)), 1, cfg, inv, w),
                           plain.decoder_layer(x_np[70:], list(range(9)), 1, cfg, inv, w)])
    assert np.abs(got - want).max() <= limit * max(1.0, np.abs(want).max())

    # head on chosen rows
    head = build_part("head", plan.head); head.load(raw, rt)
    fnorm = build_part("norm", plan.final_norm); fnorm.load(raw, rt)
    rows = torch.tensor([78, 0, 69], dtype=torch.int32, device=DEV)
    st = ResidualStream(torch.tensor(x_np, device=DEV))
    got = head.forward(fnorm.forward(st, ctx, rows=rows), ctx).cpu().numpy()
    want = plain.lm_head(x_np[[78, 0, 69]], cfg, w)
    assert got.shape == (3, V) and np.abs(got - want).max() <= limit * max(1.0, np.abs(want).max())


# ------------------------------------------------------------------ a toy mixer with state
class DecayMixer(Mixer):
    """h_t = a * h_{t-1} + (1 - a) * x_t per channel, y_t = W h_t.  Its state h is a
    record of fixed size per sequence, kept in the cache beside the keys and values
    of other layers.  Written with plain torch: it is a test's toy, not a kernel."""

    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(self.param("hidden_size"))
        self.decay_name, self.out_name = self.param("decay"), self.param("out")

    def weight_specs(self):
        return [WeightSpec(self.decay_name, (self.size,), role="vector", mean=0.0),
                WeightSpec(self.out_name, (self.size, self.size))]

    def cache_requests(self):
        return [StateRequest("h", (self.size,), "float32")]

    def load(self, tensors, rt):
        self.a = torch.sigmoid(rt.vector(tensors[self.decay_name]))
        self.w = rt.matrix(tensors[self.out_name])

    def forward(self, x, ctx, cache):
        state = cache.state("h")
        cu, slots = ctx.cu_seqlens.tolist(), ctx.slots.tolist()
        hs = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        for b, slot in enumerate(slots):
            h = state[slot].clone()
            for t in range(cu[b], cu[b + 1]):
                h = self.a * h + (1 - self.a) * x[t].float()
                hs[t] = h
            state[slot] = h
        return (hs.to(x.dtype).float() @ self.w.float().T).to(x.dtype)


def toy_plan(cfg):
    """Llama's plan with the mixer of every odd layer replaced by the toy."""
    base = llama_plan(cfg)
    layers = []
    for i, layer in enumerate(base.layers):
        if i % 2 == 1:
            layer = layer.replace(mixer=PartSpec("decay", {"hidden_size": cfg.hidden_size,
                                                           "decay": f"model.layers.{i}.decay.a",
                                                           "out": f"model.layers.{i}.decay.out.weight"}))
        layers.append(layer)
    return ModelPlan(base.hidden_size, base.vocab_size, base.embedding, tuple(layers), base.schedule,
                     base.final_norm, base.head, base.stop_tokens, base.max_position)


def plain_toy_forward(cfg, w, tokens):
    positions = list(range(len(tokens)))
    inv = plain.rope_inv_freq(cfg)
    x = plain.embed(w["model.embed_tokens.weight"], tokens)
    for i in range(cfg["num_hidden_layers"]):
        if i % 2 == 0:
            x = plain.decoder_layer(x, positions, i, cfg, inv, w)
            continue
        p = f"model.layers.{i}."
        n = plain.rms_norm(x, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        a = 1.0 / (1.0 + np.exp(-w[p + "decay.a"].astype(np.float32)))
        h = np.zeros(cfg["hidden_size"], dtype=np.float32)
        hs = np.zeros_like(n)
        for t in range(len(tokens)):
            h = a * h + (1 - a) * n[t]
            hs[t] = h
        x = x + plain.linear(hs, w[p + "decay.out.weight"])
        n2 = plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        x = x + plain.swiglu_mlp(n2, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                                 w[p + "mlp.down_proj.weight"])
    return plain.lm_head(x, cfg, w)


def test_a_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    register_part("mixer", "decay")(DecayMixer)
    arch = register_architecture(Architecture(("ToyDecayForCausalLM",), LlamaConfig.from_json, toy_plan))
    try:
        raw = dict(TINY["B"], architectures=["ToyDecayForCausalLM"], model_type="toy_decay")
        folder = str(tmp_path / "toy")
        lib.write_random_model(folder, raw, seed=5, dtype="float32", std=0.1, norm_std=0.05)
        cfg, w = plain.read_model(folder)
        model = Model.load(folder, dtype="float32", device="cuda")
        assert type(model.blocks[1].mixer) is DecayMixer
        cache = model.new_cache(max_tokens=64 * 4, max_slots=2)
        assert len(cache.groups) == 1 and cache.groups[0].storage.shape[0] == 2     # layers 0 and 2 hold keys
        p, q = make_prompts("B", [50, 20], seed=42)
        want_p, want_q = plain_toy_forward(cfg, w, p), plain_toy_forward(cfg, w, q)
        for round_ in range(2):                     # the second round reuses slots whose state is stale
            sp, sq = cache.open_sequence(), cache.open_sequence()
            got = step(model, cache, [StepEntry(sp, p[:30], list(range(30))), StepEntry(sq, q, list(range(20)))])
            got = got.cpu().numpy()
            assert_close(got[:30], want_p[:30], "float32", "toy whole")
            assert_close(got[30:], want_q, "float32", "toy second sequence")
            cache.close_sequence(sq)
            rest = [step(model, cache, [StepEntry(sp, [p[t]], [0])]).cpu().numpy() for t in range(30, 50)]
            assert_close(np.concatenate(rest), want_p[30:], "float32", "toy one by one")
            cache.close_sequence(sp)
    finally:
        unregister_architecture(arch)
        unregister_part("mixer", "decay")


# ------------------------------------------------------- the order of layers is data
def test_a_layer_named_twice_and_a_layer_that_reads_another_cache(model_folders, plain_models, tmp_path):
    name = "A"
    cfg, w = plain_models[name]
    base = llama_plan(LlamaConfig.from_json(TINY[name]))

    # layer 0 runs twice: each run has keys and values of its own
    twice = ModelPlan(base.hidden_size, base.vocab_size, base.embedding, base.layers,
                      (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0)),
                      base.final_norm, base.head, base.stop_tokens, base.max_position)
    model = Model(twice, Runtime(DEV, torch.float32)).load_tensors(tensors_of(model_folders[name]))
    cache = model.new_cache(max_tokens=64 * 2)
    assert cache.groups[0].storage.shape[0] == 3
    (p,) = make_prompts(name, [40], seed=43)
    want = plain.forward(cfg, w, p, layer_order=[0, 1, 0])
    s = cache.open_sequence()
    got = [step(model, cache, [StepEntry(s, p[:25], list(range(25)))]).cpu().numpy()]
    got += [step(model, cache, [StepEntry(s, [p[t]], [0])]).cpu().numpy() for t in range(25, 40)]
    assert_close(np.concatenate(got), want, "float32", "layer named twice")

    # a third run: layer 1's queries over the keys and values that run 0 stored
    l1 = base.layers[1]
    reader = l1.replace(mixer=PartSpec("gqa_attention", dict(l1.part("mixer").params, own_kv=False)))
    shared = ModelPlan(base.hidden_size, base.vocab_size, base.embedding, (base.layers[0], reader),
                       (ScheduleEntry(0), ScheduleEntry(1, cache=0)),
                       base.final_norm, base.head, base.stop_tokens, base.max_position)
    shared.check()
    raw = {k: v for k, v in tensors_of(model_folders[name]).items()
           if k not in ("model.layers.1.self_attn.k_proj.weight", "model.layers.1.self_attn.v_proj.weight")}
    model = Model(shared, Runtime(DEV, torch.float32)).load_tensors(raw)
    assert "model.layers.1.self_attn.k_proj.weight" not in {s.name for s in model.weight_specs()}
    cache = model.new_cache(max_tokens=64 * 2)
    assert cache.groups[0].storage.shape[0] == 1                 # one store, read by both runs

    positions = list(range(40))
    inv = plain.rope_inv_freq(cfg)
    nh, nkv, hd, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    x = plain.embed(w["model.embed_tokens.weight"], p)
    n0 = plain.rms_norm(x, w["model.layers.0.input_layernorm.weight"], eps)
    k0 = plain.rope(plain.linear(n0, w["model.layers.0.self_attn.k_proj.weight"]), positions, inv, nkv, hd)
    v0 = plain.linear(n0, w["model.layers.0.self_attn.v_proj.weight"])
    x = plain.decoder_layer(x, positions, 0, cfg, inv, w)
    n1 = plain.rms_norm(x, w["model.layers.1.input_layernorm.weight"], eps)
    q1 = plain.rope(plain.linear(n1, w["model.layers.1.self_attn.q_proj.weight"]), positions, inv, nh, hd)
    x = x + plain.linear(plain.causal_gqa_attention(q1, k0, v0, nh, nkv, hd), w["model.layers.1.self_attn.o_proj.weight"])
    n2 = plain.rms_norm(x, w["model.layers.1.post_attention_layernorm.weight"], eps)
    x = x + plain.swiglu_mlp(n2, w["model.layers.1.mlp.gate_proj.weight"], w["model.layers.1.mlp.up_proj.weight"],
                             w["model.layers.1.mlp.down_proj.weight"])
    want = plain.lm_head(x, cfg, w)
    s = cache.open_sequence()
    got = [step(model, cache, [StepEntry(s, p[:25], list(range(25)))]).cpu().numpy()]
    got += [step(model, cache, [StepEntry(s, [p[t]], [0])]).cpu().numpy() for t in range(25, 40)]
    assert_close(np.concatenate(got), want, "float32", "layer that reads another layer's cache")

    with pytest.raises(ValueError, match="does not run before"):
        ModelPlan(base.hidden_size, base.vocab_size, base.embedding, base.layers,
                  (ScheduleEntry(0, cache=1), ScheduleEntry(1)), base.final_norm, base.head).check()


# ------------------------------------------- a toy feed-forward with routing, another position encoding
class LearnedPositions(PositionEncoding):
    """x_t += P[position_t]: a table of learned absolute positions added to the
    embedded tokens; queries and keys are not rotated."""

    def __init__(self, spec):
        super().__init__(spec)
        self.n, self.size, self.name = int(self.param("max_position")), int(self.param("hidden_size")), self.param("weight")

    def weight_specs(self):
        return [WeightSpec(self.name, (self.n, self.size), role="table")]

    def load(self, tensors, rt):
        self.table = tensors[self.name].to(device=rt.device, dtype=torch.float32)

    def on_embedding(self, stream, ctx):
        stream.residual += self.table[ctx.positions.long()]


class Top1Experts(FeedForward):
    """Router logits r = R x in float32; the expert e = argmax r (first maximum)
    alone runs: y = softmax(r)[e] * D_e relu(U_e x).  Plain torch, a test's toy."""

    def __init__(self, spec):
        super().__init__(spec)
        self.h, self.i, self.e = (int(self.param(k)) for k in ("hidden_size", "intermediate_size", "n_experts"))
        self.prefix = self.param("prefix")

    def weight_specs(self):
        specs = [WeightSpec(self.prefix + "router.weight", (self.e, self.h))]
        for e in range(self.e):
            specs += [WeightSpec(f"{self.prefix}experts.{e}.up.weight", (self.i, self.h)),
                      WeightSpec(f"{self.prefix}experts.{e}.down.weight", (self.h, self.i))]
        return specs

    def load(self, tensors, rt):
        self.router = tensors[self.prefix + "router.weight"].to(device=rt.device, dtype=torch.float32)
        self.up = [rt.matrix(tensors[f"{self.prefix}experts.{e}.up.weight"]) for e in range(self.e)]
        self.down = [rt.matrix(tensors[f"{self.prefix}experts.{e}.down.weight"]) for e in range(self.e)]

    def forward(self, x, ctx):
        logits = x.float() @ self.router.T
        choice = logits.argmax(dim=1)
        weight = torch.softmax(logits, dim=1).gather(1, choice[:, None])
        out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
        for e in range(self.e):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                hidden = torch.relu(x[rows].float() @ self.up[e].float().T)
                out[rows] = hidden @ self.down[e].float().T
        return (out * weight).to(x.dtype)


N_EXPERTS = 3


def routed_plan(cfg):
    """Llama's plan with learned absolute positions instead of rotation and the
    feed-forward of layer 1 replaced by routed experts."""
    base = llama_plan(cfg)
    layers = []
    for i, layer in enumerate(base.layers):
        mixer = PartSpec(layer.part("mixer").kind, dict(layer.part("mixer").params, position=PartSpec("none")))
        ff = layer.part("feed_forward")
        if i == 1:
            ff = PartSpec("top1_experts", {"hidden_size": cfg.hidden_size, "intermediate_size": 40,
                                           "n_experts": N_EXPERTS, "prefix": f"model.layers.{i}.moe."})
        layers.append(layer.replace(mixer=mixer, feed_forward=ff))
    embedding = PartSpec(base.embedding.kind, dict(base.embedding.params, position=PartSpec(
        "learned_positions", {"max_position": 96, "hidden_size": cfg.hidden_size, "weight": "model.positions.weight"})))
    return ModelPlan(base.hidden_size, base.vocab_size, embedding, tuple(layers), base.schedule,
                     base.final_norm, base.head, base.stop_tokens, 96)


def plain_routed_forward(cfg, w, tokens):
    positions = list(range(len(tokens)))
    no_rotation = np.zeros(cfg["head_dim"] // 2)                # angle 0: cos 1, sin 0
    x = plain.embed(w["model.embed_tokens.weight"], tokens) + w["model.positions.weight"][positions].astype(np.float32)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        n = plain.rms_norm(x, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        x = (x + plain.attention_block(n, positions, p, cfg, no_rotation, w)).astype(np.float32)
        n2 = plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        if i != 1:
            x = x + plain.swiglu_mlp(n2, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                                     w[p + "mlp.down_proj.weight"])
            continue
        logits = plain.linear(n2, w[p + "moe.router.weight"])
        y = np.zeros_like(x)
        for t in range(len(tokens)):
            e = int(np.argmax(logits[t]))
            prob = np.exp(logits[t] - logits[t].max())
            prob = prob[e] / prob.sum()
            hidden = np.maximum(plain.linear(n2[t:t + 1], w[p + f"moe.experts.{e}.up.weight"]), 0)
            y[t] = prob * plain.linear(hidden, w[p + f"moe.experts.{e}.down.weight"])[0]
        x = (x + y).astype(np.float32)
    return plain.lm_head(x, cfg, w)


def test_a_routed_feed_forward_and_learned_positions_without_touching_the_library(tmp_path):
    register_part("position", "learned_positions")(LearnedPositions)
    register_part("feed_forward", "top1_experts")(Top1Experts)
    arch = register_architecture(Architecture(("ToyRoutedForCausalLM",), LlamaConfig.from_json, routed_plan))
    try:
        raw = dict(TINY["B"], architectures=["ToyRoutedForCausalLM"], model_type="toy_routed")
        folder = str(tmp_path / "routed")
        lib.write_random_model(folder, raw, seed=9, dtype="float32", std=0.1, norm_std=0.05)
        cfg, w = plain.read_model(folder)
        assert f"model.layers.1.moe.experts.{N_EXPERTS - 1}.down.weight" in w and "model.layers.1.mlp.up_proj.weight" not in w
        model = Model.load(folder, dtype="float32", device="cuda")
        assert type(model.blocks[1].feed_forward) is Top1Experts
        cache = model.new_cache(max_tokens=64 * 4, max_slots=2)
        p, q = make_prompts("B", [40, 23], seed=77)
        want_p, want_q = plain_routed_forward(cfg, w, p), plain_routed_forward(cfg, w, q)
        sp, sq = cache.open_sequence(), cache.open_sequence()
        got = step(model, cache, [StepEntry(sp, p[:25], list(range(25))), StepEntry(sq, q, list(range(23)))]).cpu().numpy()
        assert_close(got[:25], want_p[:25], "float32", "routed whole")
        assert_close(got[25:], want_q, "float32", "routed second sequence")
        rest = [step(model, cache, [StepEntry(sp, [p[t]], [0])]).cpu().numpy() for t in range(25, 40)]
        assert_close(np.concatenate(rest), want_p[25:], "float32", "routed one by one")
    finally:
        unregister_architecture(arch)
        unregister_part("position", "learned_positions")
        unregister_part("feed_forward", "top1_experts")


# ------------------------------------------- an arrangement that is not mixer + feed-forward behind two norms
class SandwichBlock(Block):
    """x += s * post1(mixer(pre1(x))); x += post2(feed_forward(pre2(x))): four norms
    and a learned scalar s per layer.  The block declares what it is made of and a
    tensor of its own; nothing in the library knows the arrangement.  The
    additions are plain torch: a test's toy."""
    sub_parts = (("pre_mixer_norm", "norm"), ("mixer", "mixer"), ("post_mixer_norm", "norm"),
                 ("pre_ff_norm", "norm"), ("feed_forward", "feed_forward"), ("post_ff_norm", "norm"))

    def weight_specs(self):
        return [WeightSpec(self.param("scalar"), (1,), role="vector", mean=1.0)]

    def load(self, tensors, rt):
        self.scalar = rt.vector(tensors[self.param("scalar")])

    def forward(self, stream, ctx, cache):
        x = self.pre_mixer_norm.forward(stream, ctx)                 # adds what the layer before left pending
        update = self.mixer.forward(x, ctx, cache)
        update = self.post_mixer_norm.forward(ResidualStream(update.float().contiguous()), ctx)
        stream.residual += self.scalar * update.float()
        x = self.pre_ff_norm.forward(stream, ctx)
        update = self.feed_forward.forward(x, ctx)
        stream.pending = self.post_ff_norm.forward(ResidualStream(update.float().contiguous()), ctx)


def sandwich_plan(cfg):
    base = llama_plan(cfg)
    layers = []
    for i, layer in enumerate(base.layers):
        p = f"model.layers.{i}."
        norm = lambda name: PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps, "weight": p + name})
        layers.append(LayerSpec(PartSpec("sandwich", {
            "pre_mixer_norm": layer.part("mixer_norm"), "mixer": layer.part("mixer"),
            "post_mixer_norm": norm("post_mixer_layernorm.weight"),
            "pre_ff_norm": layer.part("feed_forward_norm"), "feed_forward": layer.part("feed_forward"),
            "post_ff_norm": norm("post_feedforward_layernorm.weight"), "scalar": p + "layer_scalar"})))
    return ModelPlan(base.hidden_size, base.vocab_size, base.embedding, tuple(layers), base.schedule,
                     base.final_norm, base.head, base.stop_tokens, base.max_position)


def plain_sandwich_forward(cfg, w, tokens):
    positions = list(range(len(tokens)))
    inv, eps = plain.rope_inv_freq(cfg), cfg["rms_norm_eps"]
    x = plain.embed(w["model.embed_tokens.weight"], tokens)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        a = plain.attention_block(plain.rms_norm(x, w[p + "input_layernorm.weight"], eps), positions, p, cfg, inv, w)
        x = (x + w[p + "layer_scalar"].astype(np.float32) *
             plain.rms_norm(a, w[p + "post_mixer_layernorm.weight"], eps)).astype(np.float32)
        d = plain.swiglu_mlp(plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], eps),
                             w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
        x = (x + plain.rms_norm(d, w[p + "post_feedforward_layernorm.weight"], eps)).astype(np.float32)
    return plain.lm_head(x, cfg, w)


def test_a_block_with_four_norms_and_a_scalar_of_its_own(tmp_path):
    register_part("block", "sandwich")(SandwichBlock)
    arch = register_architecture(Architecture(("ToySandwichForCausalLM",), LlamaConfig.from_json, sandwich_plan))
    try:
        raw = dict(TINY["A"], architectures=["ToySandwichForCausalLM"], model_type="toy_sandwich")
        folder = str(tmp_path / "sandwich")
        lib.write_random_model(folder, raw, seed=3, dtype="float32", std=0.1, norm_std=0.05)
        cfg, w = plain.read_model(folder)
        assert w["model.layers.1.layer_scalar"].shape == (1,) and "model.layers.0.post_mixer_layernorm.weight" in w
        model = Model.load(folder, dtype="float32", device="cuda")
        names = {s.name for s in model.weight_specs()}
        assert {"model.layers.0.layer_scalar", "model.layers.1.post_feedforward_layernorm.weight"} <= names
        assert len(model.blocks[0].children()) == 6 and model.capturable
        cache = model.new_cache(max_tokens=64 * 4, max_slots=2)
        assert cache.groups[0].storage.shape[0] == 2              # the block passed its mixer's request on
        p, q = make_prompts("A", [45, 18], seed=12)
        want_p, want_q = plain_sandwich_forward(cfg, w, p), plain_sandwich_forward(cfg, w, q)
        sp, sq = cache.open_sequence(), cache.open_sequence()
        got = step(model, cache, [StepEntry(sp, p[:30], list(range(30))), StepEntry(sq, q, list(range(18)))]).cpu().numpy()
        assert_close(got[:30], want_p[:30], "float32", "sandwich whole")
        assert_close(got[30:], want_q, "float32", "sandwich second sequence")
        rest = [step(model, cache, [StepEntry(sp, [p[t]], [0])]).cpu().numpy() for t in range(30, 45)]
        assert_close(np.concatenate(rest), want_p[30:], "float32", "sandwich one by one")
        # a missing tensor of the block itself is reported like any other
        tensors = {k: v for k, v in tensors_of(folder).items() if k != "model.layers.1.layer_scalar"}
        from go_tinygrad_b200.weights import write_safetensors
        broken = tmp_path / "broken"
        broken.mkdir()
        (broken / "config.json").write_text((tmp_path / "sandwich" / "config.json").read_text())
        write_safetensors(str(broken / "model.safetensors"), tensors)
        with pytest.raises(lib.WeightError, match="layer_scalar"):
            Model.load(str(broken), dtype="float32", device="cuda")
    finally:
        unregister_architecture(arch)
        unregister_part("block", "sandwich")


# ------------------------------------------------- another layout of the rotation
def plain_rope_layout(x, positions, inv_freq, n_heads, hd, rot, interleaved):
    """The first `rot` channels of every head rotate, pair i being (i, i + rot/2) or,
    interleaved, (2i, 2i+1); the rest pass.  Written out element by element."""
    x = np.asarray(x, dtype=np.float32).reshape(len(positions), n_heads, hd)
    out = x.copy()
    for t, pos in enumerate(positions):
        for i in range(rot // 2):
            c, s = np.float32(math.cos(pos * inv_freq[i])), np.float32(math.sin(pos * inv_freq[i]))
            ia, ib = (2 * i, 2 * i + 1) if interleaved else (i, i + rot // 2)
            a, b = x[t, :, ia], x[t, :, ib]
            out[t, :, ia], out[t, :, ib] = a * c - b * s, a * s + b * c
    return out.reshape(len(positions), n_heads * hd)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name,pairing,rot", [("A", "interleaved", 16), ("A", "half", 8), ("B", "interleaved", 32)])
def test_attention_with_another_rotary_layout(model_folders, plain_models, name, pairing, rot, dtype):
    """Interleaved pairs and a rotated fraction of the head are a position
    encoding's parameters: the attention part asks the encoding for its layout and
    the general rotation kernel serves it, for prompts and for single tokens."""
    cfg, w = plain_models[name]
    raw = tensors_of(model_folders[name])
    base = llama_plan(LlamaConfig.from_json(TINY[name])).layers[1].part("mixer")
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    position = PartSpec("rotary", dict(base.params["position"].params, pairing=pairing, rotary_dim=rot))
    rt = Runtime(DEV, dtype)
    mixer = build_part("mixer", PartSpec(base.kind, dict(base.params, position=position)))
    for part in walk(mixer):
        part.load(raw, rt)
    T, head = 75, 70
    x_np = np.random.default_rng(3).standard_normal((T, cfg["hidden_size"])).astype(np.float32)
    x_act = torch.tensor(x_np, device=DEV).to(dtype)
    x_ref = x_act.float().cpu().numpy()
    cache = Cache([mixer.cache_requests()], [None], max_tokens=64 * 2, max_slots=1, dtype=dtype, device=DEV)
    slot = cache.open_sequence()
    cache.reserve(slot, T); cache.flush_tables()
    got = [mixer.forward(x_act[:head], context(rt, [head], [0], [slot]), cache.handles[0])]
    cache.advance(slot, head)
    for t in range(head, T):                                       # then token by token
        got.append(mixer.forward(x_act[t:t + 1], context(rt, [1], [t], [slot]), cache.handles[0]))
        cache.advance(slot, 1)
    got = torch.cat(got).float().cpu().numpy()

    theta = float(cfg["rope_theta"])
    inv = np.array([theta ** (-2.0 * i / rot) for i in range(rot // 2)])
    if cfg.get("rope_scaling"):
        inv = np.array(plain.rope_inv_freq(dict(cfg, head_dim=rot)))
    p = "model.layers.1.self_attn."
    positions = list(range(T))
    q = plain_rope_layout(plain.linear(x_ref, w[p + "q_proj.weight"]), positions, inv, nh, hd, rot, pairing == "interleaved")
    k = plain_rope_layout(plain.linear(x_ref, w[p + "k_proj.weight"]), positions, inv, nkv, hd, rot, pairing == "interleaved")
    v = plain.linear(x_ref, w[p + "v_proj.weight"])
    want = plain.linear(plain.causal_gqa_attention(q, k, v, nh, nkv, hd), w[p + "o_proj.weight"])
    limit = 1e-4 if dtype == torch.float32 else 4e-2
    assert np.abs(got - want).max() <= limit * max(1.0, np.abs(want).max())
    # and the layout matters: the default one gives another result
    plain_default = plain.attention_block(x_ref, positions, "model.layers.1.", cfg, plain.rope_inv_freq(cfg), w)
    assert np.abs(plain_default - want).max() > 0.1 * max(1.0, np.abs(want).max())


def test_a_rotary_layout_the_kernels_do_not_know_is_refused():
    with pytest.raises(ValueError, match="pairing"):
        build_part("position", PartSpec("rotary", {"head_dim": 16, "theta": 1e4, "pairing": "quarters"}))
    with pytest.raises(ValueError, match="rotated channels"):
        build_part("position", PartSpec("rotary", {"head_dim": 16, "theta": 1e4, "rotary_dim": 18}))
    from go_tinygrad_b200.kernels import ops
    qkv = torch.zeros((2, 64), dtype=torch.float32, device=DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    with pytest.raises(ops.KernelError, match="pairing"):
        ops.rope_kv_store(qkv, None, 4, 0, 16, None, i32([0, 0]), i32([0]), i32([0, 1]), pairing="quarters")
    with pytest.raises(ops.KernelError, match="rotary_dim"):
        ops.rope_kv_store(qkv, None, 4, 0, 16, None, i32([0, 0]), i32([0]), i32([0, 1]), rotary_dim=6 + 1)


# ------------------------------------------------- parts that talk to the host are not recorded
def test_generation_runs_a_model_that_cannot_be_captured(tmp_path):
    """The toy mixer reads device values on the host in its forward, so a step with
    it cannot be recorded as a CUDA graph; it says so (`capturable = False`) and
    the generation loop launches its decode steps in the open instead of failing
    in a capture."""
    class HostDecayMixer(DecayMixer):
        capturable = False
    register_part("mixer", "decay")(HostDecayMixer)
    arch = register_architecture(Architecture(("ToyDecayForCausalLM",), LlamaConfig.from_json, toy_plan))
    try:
        raw = dict(TINY["B"], architectures=["ToyDecayForCausalLM"], model_type="toy_decay")
        folder = str(tmp_path / "toy")
        lib.write_random_model(folder, raw, seed=5, dtype="float32", std=0.1, norm_std=0.05)
        cfg, w = plain.read_model(folder)
        model = Model.load(folder, dtype="float32", device="cuda")
        assert not model.capturable
        prompts = make_prompts("B", [12, 5], seed=8)
        got = lib.generate(model, prompts, max_new_tokens=6, stop=[])          # use_graph defaults to True
        for p, g in zip(prompts, got):
            seq = list(p)
            for tok in g.tokens:                                              # greedy against the plain toy
                assert tok == int(np.argmax(plain_toy_forward(cfg, w, seq)[-1]))
                seq.append(tok)
    finally:
        unregister_architecture(arch)
        unregister_part("mixer", "decay")


# ------------------------------------------------- layers that keep a window beside layers that keep everything
WINDOW = 37


def windowed_plan(cfg):
    """Llama's plan with every odd layer attending to the last WINDOW keys only."""
    base = llama_plan(cfg)
    layers = [layer.replace(mixer=PartSpec(layer.part("mixer").kind, dict(layer.part("mixer").params, window=WINDOW)))
              if i % 2 else layer for i, layer in enumerate(base.layers)]
    return ModelPlan(base.hidden_size, base.vocab_size, base.embedding, tuple(layers), base.schedule,
                     base.final_norm, base.head, base.stop_tokens, base.max_position)


def plain_windowed_forward(cfg, w, tokens):
    positions = list(range(len(tokens)))
    inv, eps = plain.rope_inv_freq(cfg), cfg["rms_norm_eps"]
    x = plain.embed(w["model.embed_tokens.weight"], tokens)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        n = plain.rms_norm(x, w[p + "input_layernorm.weight"], eps)
        x = (x + plain.attention_block(n, positions, p, cfg, inv, w, window=WINDOW if i % 2 else None)).astype(np.float32)
        n2 = plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
        x = (x + plain.swiglu_mlp(n2, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                                  w[p + "mlp.down_proj.weight"])).astype(np.float32)
    return plain.lm_head(x, cfg, w)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_windowed_layers_beside_full_layers(model_folders, plain_models, name, dtype):
    """Mixers differ layer by layer (every odd one sees a window of 37 keys), so the
    cache has two groups with storage of their own; prompts longer than the window,
    a prompt cut where the window's edge falls inside a chunk, and single tokens
    whose window has slid past the first page, which the windowed group has then
    given back (and takes again for its third page)."""
    arch = register_architecture(Architecture(("ToyWindowForCausalLM",), LlamaConfig.from_json, windowed_plan))
    try:
        cfg, w = plain_models[name]
        raw = dict(TINY[name], architectures=["ToyWindowForCausalLM"])
        model = Model(arch.plan(arch.read_config(raw)), Runtime(DEV, getattr(torch, dtype))).load_tensors(
            tensors_of(model_folders[name]))
        cache = model.new_cache(max_tokens=64 * 6, max_slots=2)
        n_layers = cfg["num_hidden_layers"]
        assert len(cache.groups) == 2
        assert sorted(g.storage.shape[0] for g in cache.groups) == sorted([(n_layers + 1) // 2, n_layers // 2])
        assert {g.request.window for g in cache.groups} == {None, WINDOW}
        p, q = make_prompts(name, [130, 50], seed=51)
        want_p, want_q = plain_windowed_forward(cfg, w, p), plain_windowed_forward(cfg, w, q)
        sp, sq = cache.open_sequence(), cache.open_sequence()
        got = step(model, cache, [StepEntry(sp, p[:80], list(range(80))), StepEntry(sq, q, list(range(50)))])
        got = got.float().cpu().numpy()
        assert_close(got[:80], want_p[:80], dtype, f"{name} windowed: whole")
        assert_close(got[80:], want_q, dtype, f"{name} windowed: second sequence")
        cache.close_sequence(sq)
        got = step(model, cache, [StepEntry(sp, p[80:110], list(range(30)))]).float().cpu().numpy()   # a chunk after the prompt
        assert_close(got, want_p[80:110], dtype, f"{name} windowed: chunk")
        # the windowed group has given back the first page (keys 0..63 are behind every later
        # window); the other group keeps it.  Whatever lies in pages no sequence holds, and in
        # the page given back once another sequence writes it, must not reach a result
        win = next(g for g in cache.groups if g.request.window == WINDOW)
        keeps = next(g for g in cache.groups if g.request.window is None)
        assert win.pages_of[sp][0] == -1 and all(x >= 0 for x in win.pages_of[sp][1:]) and min(keeps.pages_of[sp]) >= 0
        assert win.pool.n_free == keeps.pool.n_free + 1
        held = [x for x in win.pages_of[sp] if x >= 0]
        loose = [x for x in range(win.pool.n_pages) if x not in held]
        win.storage[:, loose] = 3.0e4           # finite, and large enough to wreck any sum it entered
        rest = [step(model, cache, [StepEntry(sp, [p[t]], [0])]).float().cpu().numpy() for t in range(110, 130)]
        assert_close(np.concatenate(rest), want_p[110:], dtype, f"{name} windowed: one by one")
        # the window matters: without it the logits differ visibly
        full = plain.forward(cfg, w, p)
        assert np.abs(full[100:] - want_p[100:]).max() > 0.05 * np.abs(want_p).max()
    finally:
        unregister_architecture(arch)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("use_graph", [True, False])
def test_generation_through_windowed_layers_gives_pages_back_under_recorded_steps(model_folders, plain_models, use_graph,
                                                                                   dtype):
    """Greedy generation far past the window through the toy model above: the
    windowed group gives pages back while decode steps are replayed from a recording,
    sequences of unequal lengths end at different times, and every token is the plain
    implementation's choice from the same prefix; the cache ends empty."""
    name = "A"
    arch = register_architecture(Architecture(("ToyWindowForCausalLM",), LlamaConfig.from_json, windowed_plan))
    try:
        cfg, w = plain_models[name]
        raw = dict(TINY[name], architectures=["ToyWindowForCausalLM"])
        model = Model(arch.plan(arch.read_config(raw)), Runtime(DEV, getattr(torch, dtype))).load_tensors(
            tensors_of(model_folders[name]))
        prompts = make_prompts(name, [70, 9, 131], seed=61)
        limits = [150, 40, 90]
        cache = model.new_cache(max_tokens=64 * 12, max_slots=3)
        released = []
        real_advance = cache.advance

        def watching(slot, n):
            real_advance(slot, n)
            win = next(g for g in cache.groups if g.request.window == WINDOW)
            released.append(sum(1 for p in win.pages_of[slot] if p < 0))
        cache.advance = watching
        out = lib.generate(model, prompts, limits, stop=[], cache=cache, use_graph=use_graph)
        assert max(released) >= 2                      # pages did go back while the batch ran
        for p, r, n in zip(prompts, out, limits):
            assert len(r.tokens) == n
            # one pass of the plain implementation over prompt and answer: at every place the
            # token that was chosen must be the maximum there (or within rounding of it)
            logits = plain_windowed_forward(cfg, w, list(p) + r.tokens[:-1]).astype(np.float64)
            for t, tok in enumerate(r.tokens):
                row = logits[len(p) - 1 + t]
                slack = (1e-4 if dtype == "float32" else 5e-2) * max(1.0, np.abs(row).max())
                assert row[tok] >= row.max() - slack, (len(p), t, tok, int(row.argmax()))
        assert cache.open_slots() == [] and all(f == cache.n_pages for f in cache.free_pages())
    finally:
        unregister_architecture(arch)
