"""Each part alone against its plain function, and toy architectures assembled from parts that the test defines:
a mixer with state of its own, a feed-forward with routing, another position encoding."""

import numpy as np
import pytest
import torch

import plain_model
from tau_rs_b200 import Engine, StepEntry, load_model, write_random_model
from tau_rs_b200.cache import SequenceCache
from tau_rs_b200.config import (AttentionSpec, BlockSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry, SwiGLUSpec,
                                register_architecture, unregister_architecture)
from tau_rs_b200.engine.batch import StepLayout, fill_step, step_views
from tau_rs_b200.parts import (CacheNeed, FeedForward, Mixer, Part, build, register_feed_forward, register_mixer, register_position,
                               unregister)
from tau_rs_b200.weights import TensorSpec, random_tensors

pytestmark = pytest.mark.gpu
DEVICE = torch.device("cuda:0")
TOLERANCE = {torch.float32: 2e-5, torch.bfloat16: 1.5e-2}


def error(found, wanted):
    return float((found.double().cpu() - wanted.double()).abs().max() / wanted.double().abs().max())


def fill(part, dtype, seed=0, jitter=0.1):
    """Random weights for one part; returns them (as float32 on the host, rounded through the part's dtype)."""
    plain = {}
    for name, tensor, spec in random_tensors(part.tensor_specs(), seed, jitter):
        stored = tensor.to(dtype) if spec.role == "matrix" else tensor
        part.assign(name, stored.to(DEVICE))
        plain[name] = stored.float()
    part.finalize_weights()
    return plain


def rounding(dtype):
    return plain_model.bfloat16_rounding if dtype == torch.bfloat16 else plain_model.no_rounding


def single_sequence_step(cache, slot, count, start=0):
    entry = StepEntry(slot, [0] * count, [])
    cache.reserve(slot, start + count)
    layout = StepLayout(count, 1, 0, {group: (start + count + 63) // 64 for group in cache.kv})
    staged = np.zeros(layout.total, dtype=np.int32)
    fill_step(layout, staged, [entry], [start], cache)
    step = step_views(layout, torch.from_numpy(staged).to(DEVICE), count, start + count, count == 1)
    cache.advance(slot, start + count)
    return step


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    spec = NormSpec(width=200, eps=3e-4)
    part = build("norm", spec, name="n.weight", dtype=dtype, device=DEVICE)
    plain = fill(part, dtype)
    x = torch.randn(9, 200).to(dtype)
    branch = torch.randn(9, 200).to(dtype)
    assert error(part.forward(x.to(DEVICE)), plain_model.rms_norm(x.float(), plain["n.weight"], 3e-4, rounding(dtype))) < TOLERANCE[dtype]
    residual = x.to(DEVICE).clone()
    normed = part.add_forward(branch.to(DEVICE), residual)
    summed = rounding(dtype)(x.float() + branch.float())
    assert torch.equal(residual.float().cpu(), summed)
    assert error(normed, plain_model.rms_norm(summed, plain["n.weight"], 3e-4, rounding(dtype))) < TOLERANCE[dtype]


def test_rotary_tables_part():
    spec = PositionSpec(rotary_dim=48, theta=50000.0, max_positions=300)
    part = build("position", spec, device=DEVICE)
    part.finalize_weights()
    cos, sin = plain_model.rope_tables(48, 50000.0, 300)
    assert torch.equal(part.cos.cpu(), cos) and torch.equal(part.sin.cpu(), sin)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    spec = SwiGLUSpec(hidden=72, intermediate=200)
    part = build("feed_forward", spec, prefix="ff", dtype=dtype, device=DEVICE)
    plain = fill(part, dtype)
    x = torch.randn(70, 72).to(dtype)
    found = part.forward(x.to(DEVICE), None)
    assert error(found, plain_model.swiglu(x.float(), plain, "ff", rounding(dtype))) < TOLERANCE[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,groups,width,bias", [(6, 2, 32, True), (3, 3, 80, False)])
def test_attention_part_whole_then_stepwise(dtype, heads, groups, width, bias):
    hidden = 56
    spec = AttentionSpec(hidden=hidden, n_heads=heads, n_kv_heads=groups, head_dim=width, bias=bias, softmax_scale=width ** -0.5,
                         qk_norm=NormSpec(width=width, eps=1e-5), position=PositionSpec(rotary_dim=width, theta=1e4, max_positions=256))
    part = build("mixer", spec, prefix="attn", dtype=dtype, device=DEVICE)
    plain = fill(part, dtype)
    config = plain_model.PlainConfig(vocab_size=1, hidden_size=hidden, intermediate_size=1, num_hidden_layers=1, num_attention_heads=heads,
                                     num_key_value_heads=groups, head_dim=width, attention_bias=bias, rms_norm_eps=1e-5, rope_theta=1e4,
                                     max_position_embeddings=256, tie_word_embeddings=True)
    cos, sin = plain_model.rope_tables(width, 1e4, 256)
    x = torch.randn(90, hidden).to(dtype)
    wanted = plain_model.attention_mixer(x.float(), plain, "attn", config, cos, sin, rounding(dtype))
    cache = SequenceCache({"g": (part.cache_need(), 1)}, 256, 256, dtype, DEVICE)
    slot = cache.open()
    view = cache.layer_view("g", 0)
    found = [part.forward(x[:70].to(DEVICE), single_sequence_step(cache, slot, 70), view, True)]
    for position in range(70, 90):
        found.append(part.forward(x[position : position + 1].to(DEVICE), single_sequence_step(cache, slot, 1, position), view, True))
    assert error(torch.cat(found), wanted) < TOLERANCE[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_part(dtype):
    hidden = 48
    norm = NormSpec(width=hidden, eps=1e-6)
    attention = AttentionSpec(hidden=hidden, n_heads=4, n_kv_heads=1, head_dim=16, bias=False, softmax_scale=0.25,
                              qk_norm=NormSpec(width=16, eps=1e-6), position=PositionSpec(rotary_dim=16, theta=1e4, max_positions=128))
    spec = BlockSpec(prefix="model.layers.0", mixer=attention, feed_forward=SwiGLUSpec(hidden=hidden, intermediate=100),
                     mixer_norm=norm, feed_forward_norm=norm)
    part = build("block", spec, dtype=dtype, device=DEVICE)
    plain = fill(part, dtype)
    config = plain_model.PlainConfig(vocab_size=1, hidden_size=hidden, intermediate_size=100, num_hidden_layers=1, num_attention_heads=4,
                                     num_key_value_heads=1, head_dim=16, attention_bias=False, rms_norm_eps=1e-6, rope_theta=1e4,
                                     max_position_embeddings=128, tie_word_embeddings=True)
    cos, sin = plain_model.rope_tables(16, 1e4, 128)
    x = torch.randn(33, hidden).to(dtype)
    wanted = plain_model.decoder_block(x.float(), plain, "model.layers.0", config, cos, sin, rounding(dtype))
    cache = SequenceCache({"g": (part.cache_need(), 1)}, 128, 128, dtype, DEVICE)
    slot = cache.open()
    residual, branch = part.forward(x.to(DEVICE).clone(), None, single_sequence_step(cache, slot, 33), cache.layer_view("g", 0), True)
    found = rounding(dtype)(residual.float().cpu() + branch.float().cpu())
    assert error(found, wanted) < TOLERANCE[dtype]


# ------------------------------------------------------------------------------------------------
# A toy mixer with state of its own, defined here, registered, built and stepped without touching the library.
class DecaySpec:
    kind = "toy_decay"

    def __init__(self, hidden, decay):
        self.hidden, self.decay = hidden, decay

    def __eq__(self, other):
        return isinstance(other, DecaySpec) and (self.hidden, self.decay) == (other.hidden, other.decay)

    def __hash__(self):
        return hash((self.hidden, self.decay))


class DecayMixer(Mixer):
    """`s_t = decay * s_{t-1} + x_t W^T`, `y_t = s_t`: one vector of state per sequence, whatever its length."""

    def __init__(self, spec, prefix, dtype, device):
        self.spec, self.prefix, self.dtype = spec, prefix, dtype
        self.weight = None

    def cache_need(self):
        return CacheNeed("state", state_shape=(self.spec.hidden,), state_dtype=torch.float32)

    def tensor_specs(self):
        return {f"{self.prefix}.mix.weight": TensorSpec((self.spec.hidden, self.spec.hidden), role="matrix", std=0.1)}

    def assign(self, name, tensor):
        self.weight = tensor

    def forward(self, hidden, step, cache, writes_cache):
        projected = hidden.float() @ self.weight.float().t()
        if step.all_single:   # one token per sequence: everything stays on the device, so the step can be captured in a graph
            slots = step.seq_slot.long()
            state = cache.state.index_select(0, slots) * self.spec.decay + projected
            cache.state.index_copy_(0, slots, state)
            return state.to(hidden.dtype)
        out = torch.empty_like(projected)
        bounds, slots = step.cu_seqlens.cpu().tolist(), step.seq_slot.cpu().tolist()
        for index, slot in enumerate(slots):
            state = cache.state[slot]
            for row in range(bounds[index], bounds[index + 1]):
                state.mul_(self.spec.decay).add_(projected[row])
                out[row] = state
        return out.to(hidden.dtype)


def toy_spec(config) -> ModelSpec:
    hidden = config["hidden_size"]
    norm = NormSpec(width=hidden, eps=config["eps"])
    attention = AttentionSpec(hidden=hidden, n_heads=4, n_kv_heads=2, head_dim=16, bias=False, softmax_scale=0.25,
                              qk_norm=None, position=PositionSpec(rotary_dim=8, theta=100.0, max_positions=config["max_positions"]))
    feed = SwiGLUSpec(hidden=hidden, intermediate=config["intermediate_size"])
    blocks = (
        BlockSpec("toy.layers.0", DecaySpec(hidden, 0.9), feed, norm, norm),
        BlockSpec("toy.layers.1", attention, feed, norm, norm),
    )
    schedule = (
        ScheduleEntry(layer=0, cache_group="decay", cache_layer=0),
        ScheduleEntry(layer=1, cache_group="keys", cache_layer=0),
        ScheduleEntry(layer=0, cache_group="decay", cache_layer=1),                    # the same weights again, state of its own
        ScheduleEntry(layer=1, cache_group="keys", cache_layer=0, writes_cache=False), # reads the keys the earlier run wrote
    )
    return ModelSpec(architecture="ToyForCausalLM", vocab_size=config["vocab_size"], hidden=hidden, max_positions=config["max_positions"],
                     embedding_name="toy.embed.weight", blocks=blocks, schedule=schedule, final_norm=norm,
                     final_norm_name="toy.norm.weight", head_name="toy.head.weight", tie_head=False)


@pytest.fixture
def toy_architecture():
    register_mixer("toy_decay")(DecayMixer)
    register_architecture("ToyForCausalLM", "toy", lambda raw: raw, toy_spec)
    yield
    unregister_architecture("ToyForCausalLM")
    unregister("mixer", "toy_decay")


def test_a_toy_mixer_with_state_is_registered_built_and_stepped(toy_architecture, tmp_path):
    config = {"architectures": ["ToyForCausalLM"], "model_type": "toy", "hidden_size": 40, "intermediate_size": 72, "vocab_size": 97,
              "max_positions": 200, "eps": 1e-5}
    folder = str(tmp_path / "toy")
    write_random_model(folder, config, seed=4, norm_jitter=0.1, storage="float32")
    model = load_model(folder, "float32", DEVICE)
    assert set(model.cache_groups()) == {"decay", "keys"}
    assert model.cache_groups()["decay"][1] == 2 and model.cache_groups()["keys"][1] == 1
    engine = Engine(model, 64 * 6)
    # Decode steps are captured: the warm-up run before a capture advances the state once, and it is put back before the replay.
    assert engine.use_graphs
    DecayMixer.capturable = False
    try:
        assert not Engine(load_model(folder, "float32", DEVICE), 64).use_graphs      # a part that cannot be captured says so
    finally:
        DecayMixer.capturable = True
    rng = np.random.default_rng(0)
    requests = [rng.integers(0, 97, size=length).tolist() for length in (70, 9, 33)]

    def whole(tokens):
        slot = engine.open_sequence()
        logits = engine.step([StepEntry(slot, tokens, list(range(len(tokens))))]).cpu().clone()
        engine.close_sequence(slot)
        return logits

    alone = [whole(tokens) for tokens in requests]
    # The same requests as a batch of unequal lengths: prompts first, then token by token, on slots used before.
    slots = [engine.open_sequence() for _ in requests]
    prompt_lengths = [40, 5, 33]
    logits = engine.step([StepEntry(slot, tokens[:cut], [cut - 1]) for slot, tokens, cut in zip(slots, requests, prompt_lengths)]).cpu()
    for row, cut in enumerate(prompt_lengths):
        assert error(logits[row], alone[row][cut - 1]) < 1e-4
    for offset in range(4):
        live = [index for index in range(3) if prompt_lengths[index] + offset < len(requests[index])]
        logits = engine.step([StepEntry(slots[i], [requests[i][prompt_lengths[i] + offset]], [0]) for i in live]).cpu()
        for row, i in enumerate(live):
            assert error(logits[row], alone[i][prompt_lengths[i] + offset]) < 1e-4
    for slot in slots:
        engine.close_sequence(slot)
    engine.cache.check()
    # Independent check of the whole model against plain functions for its parts.
    weights = plain_model.read_plain_weights(folder)
    tokens = requests[0]
    hidden = plain_model.embedding(weights["toy.embed.weight"], tokens)
    cos, sin = plain_model.rope_tables(8, 100.0, 200)
    keys_seen = {}

    def decay_run(x, prefix):
        projected = x @ weights[f"{prefix}.self_attn.mix.weight"].t()
        state, rows = torch.zeros(40), []
        for row in projected:
            state = 0.9 * state + row
            rows.append(state)
        return torch.stack(rows)

    def attention_run(x, prefix, reuse):
        count = x.shape[0]
        q = (x @ weights[f"{prefix}.self_attn.q_proj.weight"].t()).view(count, 4, 16)
        rotate = lambda t: torch.cat([plain_model.apply_rope(t[..., :8], cos[:count], sin[:count], plain_model.no_rounding), t[..., 8:]], dim=-1)
        if not reuse:
            k = (x @ weights[f"{prefix}.self_attn.k_proj.weight"].t()).view(count, 2, 16)
            v = (x @ weights[f"{prefix}.self_attn.v_proj.weight"].t()).view(count, 2, 16)
            keys_seen["k"], keys_seen["v"] = rotate(k), v
        context = plain_model.causal_attention(rotate(q), keys_seen["k"], keys_seen["v"], plain_model.no_rounding)
        return context.reshape(count, 64) @ weights[f"{prefix}.self_attn.o_proj.weight"].t()

    for layer, reuse in ((0, False), (1, False), (0, False), (1, True)):
        prefix = f"toy.layers.{layer}"
        normed = plain_model.rms_norm(hidden, weights[f"{prefix}.input_layernorm.weight"], 1e-5, plain_model.no_rounding)
        hidden = hidden + (decay_run(normed, prefix) if layer == 0 else attention_run(normed, prefix, reuse))
        normed = plain_model.rms_norm(hidden, weights[f"{prefix}.post_attention_layernorm.weight"], 1e-5, plain_model.no_rounding)
        hidden = hidden + plain_model.swiglu(normed, weights, f"{prefix}.mlp", plain_model.no_rounding)
    expected = plain_model.rms_norm(hidden, weights["toy.norm.weight"], 1e-5, plain_model.no_rounding) @ weights["toy.head.weight"].t()
    assert error(alone[0], expected) < 1e-4


# ------------------------------------------------------------------------------------------------
# A feed-forward with routing and another position encoding, defined here: layers of one model take different
# feed-forwards and different position encodings, chosen by their descriptions alone.
class RoutedSpec:
    kind = "toy_routed"

    def __init__(self, hidden, widths, top):
        self.hidden, self.widths, self.top = hidden, tuple(widths), top       # one SwiGLU expert per width

    def __eq__(self, other):
        return isinstance(other, RoutedSpec) and (self.hidden, self.widths, self.top) == (other.hidden, other.widths, other.top)

    def __hash__(self):
        return hash((self.hidden, self.widths, self.top))


class RoutedFeedForward(FeedForward):
    """Router logits in 32-bit, softmax over all experts, the `top` largest renormalised, experts of unequal widths."""

    def __init__(self, spec, prefix, dtype, device):
        self.spec, self.prefix = spec, prefix
        self.tensors = {}

    def tensor_specs(self):
        specs = {f"{self.prefix}.router.weight": TensorSpec((len(self.spec.widths), self.spec.hidden), role="vector", std=0.5)}
        for index, width in enumerate(self.spec.widths):
            specs[f"{self.prefix}.experts.{index}.gate_proj.weight"] = TensorSpec((width, self.spec.hidden), std=0.1)
            specs[f"{self.prefix}.experts.{index}.up_proj.weight"] = TensorSpec((width, self.spec.hidden), std=0.1)
            specs[f"{self.prefix}.experts.{index}.down_proj.weight"] = TensorSpec((self.spec.hidden, width), std=0.1)
        return specs

    def assign(self, name, tensor):
        self.tensors[name] = tensor

    def forward(self, hidden, step):
        return routed_feed_forward(hidden.float(), self.tensors, self.prefix, self.spec).to(hidden.dtype)

    def bytes_read_per_step(self, dtype):
        """A token reads the router and its `top` experts; the largest experts bound what a step of one token reads."""
        element = torch.empty((), dtype=dtype).element_size()
        largest = sorted(self.spec.widths, reverse=True)[: self.spec.top]
        return len(self.spec.widths) * self.spec.hidden * 4 + sum(3 * width * self.spec.hidden * element for width in largest)


def routed_feed_forward(x, weights, prefix, spec):
    scores = torch.softmax(x @ weights[f"{prefix}.router.weight"].float().t(), dim=-1)
    best, chosen = scores.topk(spec.top, dim=-1)
    best = best / best.sum(dim=-1, keepdim=True)
    out = torch.zeros_like(x)
    for index in range(len(spec.widths)):
        gate = x @ weights[f"{prefix}.experts.{index}.gate_proj.weight"].float().t()
        up = x @ weights[f"{prefix}.experts.{index}.up_proj.weight"].float().t()
        expert = (torch.nn.functional.silu(gate) * up) @ weights[f"{prefix}.experts.{index}.down_proj.weight"].float().t()
        share = (best * (chosen == index)).sum(dim=-1, keepdim=True)      # zero where the expert was not chosen
        out += share * expert
    return out


class SlowedRotarySpec:
    """Rotation angles `position / slowdown * theta^(-i / rotary_dim)`: the attention part needs only `rotary_dim` here."""
    kind = "toy_slowed_rotary"

    def __init__(self, rotary_dim, theta, slowdown, max_positions):
        self.rotary_dim, self.theta, self.slowdown, self.max_positions = rotary_dim, theta, slowdown, max_positions

    def __eq__(self, other):
        return isinstance(other, SlowedRotarySpec) and vars(self) == vars(other)

    def __hash__(self):
        return hash(tuple(sorted(vars(self).items())))


def slowed_tables(spec):
    inverse = torch.tensor([spec.theta ** (-index / spec.rotary_dim) for index in range(0, spec.rotary_dim, 2)], dtype=torch.float32)
    angles = (torch.arange(spec.max_positions, dtype=torch.float32) / spec.slowdown)[:, None] * inverse[None, :]
    return torch.cos(angles), torch.sin(angles)


class SlowedRotary(Part):
    """A position encoding is a part that holds `cos` and `sin`, `[max_positions, rotary_dim / 2]` in float32, once its weights are final."""

    def __init__(self, spec, device):
        self.spec, self.device = spec, device
        self.cos = self.sin = None

    def finalize_weights(self):
        cos, sin = slowed_tables(self.spec)
        self.cos, self.sin = cos.contiguous().to(self.device), sin.contiguous().to(self.device)


def routed_spec(config) -> ModelSpec:
    hidden = config["hidden_size"]
    norm = NormSpec(width=hidden, eps=config["eps"])
    slowed = AttentionSpec(hidden=hidden, n_heads=3, n_kv_heads=1, head_dim=32, bias=True, softmax_scale=32 ** -0.5,
                           qk_norm=NormSpec(width=32, eps=config["eps"]),
                           position=SlowedRotarySpec(rotary_dim=16, theta=500.0, slowdown=config["slowdown"], max_positions=config["max_positions"]))
    usual = AttentionSpec(hidden=hidden, n_heads=2, n_kv_heads=2, head_dim=16, bias=False, softmax_scale=0.25, qk_norm=None,
                          position=PositionSpec(rotary_dim=16, theta=100.0, max_positions=config["max_positions"]))
    blocks = (
        BlockSpec("toy.layers.0", slowed, RoutedSpec(hidden, config["expert_widths"], config["experts_per_token"]), norm, norm),
        BlockSpec("toy.layers.1", usual, SwiGLUSpec(hidden=hidden, intermediate=config["intermediate_size"]), norm, norm),
    )
    schedule = (ScheduleEntry(layer=0, cache_group="wide", cache_layer=0), ScheduleEntry(layer=1, cache_group="narrow", cache_layer=0))
    return ModelSpec(architecture="ToyRoutedForCausalLM", vocab_size=config["vocab_size"], hidden=hidden, max_positions=config["max_positions"],
                     embedding_name="toy.embed.weight", blocks=blocks, schedule=schedule, final_norm=norm,
                     final_norm_name="toy.norm.weight", head_name="toy.head.weight", tie_head=True)


@pytest.fixture
def routed_architecture():
    register_feed_forward("toy_routed")(RoutedFeedForward)
    register_position("toy_slowed_rotary")(SlowedRotary)
    register_architecture("ToyRoutedForCausalLM", "toy_routed", lambda raw: raw, routed_spec)
    yield
    unregister_architecture("ToyRoutedForCausalLM")
    unregister("feed_forward", "toy_routed")
    unregister("position", "toy_slowed_rotary")


def test_a_toy_routed_feed_forward_and_another_position_encoding(routed_architecture, tmp_path):
    config = {"architectures": ["ToyRoutedForCausalLM"], "model_type": "toy_routed", "hidden_size": 24, "intermediate_size": 40,
              "vocab_size": 61, "max_positions": 160, "eps": 1e-5, "expert_widths": [16, 40, 8], "experts_per_token": 2, "slowdown": 4.0}
    folder = str(tmp_path / "routed")
    write_random_model(folder, config, seed=6, norm_jitter=0.1, storage="float32")
    model = load_model(folder, "float32", DEVICE)
    assert set(model.cache_groups()) == {"wide", "narrow"}
    engine = Engine(model, 64 * 5)
    rng = np.random.default_rng(1)
    requests = [rng.integers(0, 61, size=length).tolist() for length in (80, 21)]

    # The plain statement of the model, part by part, from the files.
    weights = plain_model.read_plain_weights(folder)
    spec = routed_spec(config)

    def attention_run(x, prefix, attention, cos, sin):
        count, rot = x.shape[0], attention.position.rotary_dim
        bias = lambda name: weights[f"{prefix}.{name}.bias"] if attention.bias else 0.0
        q = (x @ weights[f"{prefix}.q_proj.weight"].t() + bias("q_proj")).view(count, attention.n_heads, attention.head_dim)
        k = (x @ weights[f"{prefix}.k_proj.weight"].t() + bias("k_proj")).view(count, attention.n_kv_heads, attention.head_dim)
        v = (x @ weights[f"{prefix}.v_proj.weight"].t() + bias("v_proj")).view(count, attention.n_kv_heads, attention.head_dim)
        if attention.qk_norm is not None:
            q = plain_model.rms_norm(q, weights[f"{prefix}.q_norm.weight"], attention.qk_norm.eps, plain_model.no_rounding)
            k = plain_model.rms_norm(k, weights[f"{prefix}.k_norm.weight"], attention.qk_norm.eps, plain_model.no_rounding)
        rotate = lambda t: torch.cat([plain_model.apply_rope(t[..., :rot], cos[:count], sin[:count], plain_model.no_rounding), t[..., rot:]], dim=-1)
        context = plain_model.causal_attention(rotate(q), rotate(k), v, plain_model.no_rounding)
        return context.reshape(count, -1) @ weights[f"{prefix}.o_proj.weight"].t() + bias("o_proj")   # one flag for all four projections

    def expected(tokens):
        hidden = plain_model.embedding(weights["toy.embed.weight"], tokens)
        tables = (slowed_tables(spec.blocks[0].mixer.position), plain_model.rope_tables(16, 100.0, 160))
        for layer, block in enumerate(spec.blocks):
            prefix = f"toy.layers.{layer}"
            normed = plain_model.rms_norm(hidden, weights[f"{prefix}.input_layernorm.weight"], 1e-5, plain_model.no_rounding)
            hidden = hidden + attention_run(normed, f"{prefix}.self_attn", block.mixer, *tables[layer])
            normed = plain_model.rms_norm(hidden, weights[f"{prefix}.post_attention_layernorm.weight"], 1e-5, plain_model.no_rounding)
            hidden = hidden + (routed_feed_forward(normed, weights, f"{prefix}.mlp", block.feed_forward) if layer == 0
                               else plain_model.swiglu(normed, weights, f"{prefix}.mlp", plain_model.no_rounding))
        return plain_model.rms_norm(hidden, weights["toy.norm.weight"], 1e-5, plain_model.no_rounding) @ weights["toy.embed.weight"].t()

    wanted = [expected(tokens) for tokens in requests]
    # Whole, then as a batch of unequal prompts followed by single tokens.
    for tokens, reference in zip(requests, wanted):
        slot = engine.open_sequence()
        logits = engine.step([StepEntry(slot, tokens, list(range(len(tokens))))]).cpu()
        engine.close_sequence(slot)
        assert error(logits, reference) < 1e-4
    slots = [engine.open_sequence() for _ in requests]
    cuts = [70, 15]
    logits = engine.step([StepEntry(slot, tokens[:cut], [cut - 1]) for slot, tokens, cut in zip(slots, requests, cuts)]).cpu()
    for row, cut in enumerate(cuts):
        assert error(logits[row], wanted[row][cut - 1]) < 1e-4
    for offset in range(6):
        logits = engine.step([StepEntry(slots[i], [requests[i][cuts[i] + offset]], [0]) for i in range(2)]).cpu()
        for i in range(2):
            assert error(logits[i], wanted[i][cuts[i] + offset]) < 1e-4
    for slot in slots:
        engine.close_sequence(slot)
    engine.cache.check()
    # The roofline's bytes follow what the routed part says it reads: two of its three experts, not all of them.
    every_tensor = sum(tensor.numel() * tensor.element_size() for tensor in model.blocks[0].feed_forward.tensors.values())
    told = model.blocks[0].feed_forward.bytes_read_per_step(torch.float32)
    assert told == 3 * 24 * 4 + 3 * (40 + 16) * 24 * 4 < every_tensor
    assert model.weight_bytes() == (sum(block.bytes_read_per_step(torch.float32) for block in model.blocks)
                                    + model.final_norm.bytes_read_per_step(torch.float32) + 61 * 24 * 4)
    assert model.blocks[1].feed_forward.bytes_read_per_step(torch.float32) == 3 * 40 * 24 * 4      # a dense part reads every tensor
    # The slowdown is felt: the same weights with the usual tables give other logits.
    usual = plain_model.rope_tables(16, 500.0, 160)
    assert not torch.allclose(torch.stack(slowed_tables(spec.blocks[0].mixer.position)), torch.stack(usual))


# ---- a position encoding that acts at the embedding -------------------------------------------------------------------
class LearnedPositionsSpec:
    kind = "toy_learned_positions"

    def __init__(self, hidden, max_positions, name):
        self.hidden, self.max_positions, self.name = hidden, max_positions, name

    def __eq__(self, other):
        return isinstance(other, LearnedPositionsSpec) and vars(self) == vars(other)

    def __hash__(self):
        return hash(tuple(sorted(vars(self).items())))


class LearnedPositions(Part):
    """`h_t = E[token_t] + P[position_t]`: a table of one vector per position, added to the embedded tokens before the first
    block.  A model names it as `ModelSpec.input_position`; its part offers `add_to(hidden, step)`."""

    def __init__(self, spec, device):
        self.spec, self.table = spec, None

    def tensor_specs(self):
        return {self.spec.name: TensorSpec((self.spec.max_positions, self.spec.hidden), role="matrix", std=0.5)}

    def assign(self, name, tensor):
        self.table = tensor

    def add_to(self, hidden, step):
        hidden.add_(self.table.index_select(0, step.positions.long()).to(hidden.dtype))


def absolute_spec(config) -> ModelSpec:
    """Dense Qwen3 blocks without any rotation, positions learned and added at the embedding."""
    hidden = config["hidden_size"]
    norm = NormSpec(width=hidden, eps=config["eps"])
    attention = AttentionSpec(hidden=hidden, n_heads=4, n_kv_heads=2, head_dim=16, bias=False, softmax_scale=0.25,
                              qk_norm=NormSpec(width=16, eps=config["eps"]), position=None)
    feed = SwiGLUSpec(hidden=hidden, intermediate=config["intermediate_size"])
    blocks = tuple(BlockSpec(f"model.layers.{index}", attention, feed, norm, norm) for index in range(2))
    schedule = tuple(ScheduleEntry(layer=index, cache_group="attention", cache_layer=index) for index in range(2))
    return ModelSpec(architecture="ToyAbsoluteForCausalLM", vocab_size=config["vocab_size"], hidden=hidden, max_positions=config["max_positions"],
                     embedding_name="model.embed_tokens.weight", blocks=blocks, schedule=schedule, final_norm=norm,
                     final_norm_name="model.norm.weight", head_name="lm_head.weight", tie_head=True,
                     input_position=LearnedPositionsSpec(hidden, config["max_positions"], "model.embed_positions.weight"))


@pytest.mark.parametrize("dtype,tolerance", [("float32", 1e-4), ("bfloat16", 2e-2)])
def test_a_toy_position_encoding_that_acts_at_the_embedding(dtype, tolerance, tmp_path):
    """Learned absolute positions, registered, built and stepped without a change to the library: whole prompts, an unequal
    batch and single tokens (through captured graphs on the GPU), against the plain blocks with a rotation of angle zero."""
    config = {"architectures": ["ToyAbsoluteForCausalLM"], "model_type": "toy_absolute", "hidden_size": 64, "intermediate_size": 96,
              "vocab_size": 83, "max_positions": 128, "eps": 1e-6}
    register_position("toy_learned_positions")(LearnedPositions)
    register_architecture("ToyAbsoluteForCausalLM", "toy_absolute", lambda raw: raw, absolute_spec)
    try:
        folder = str(tmp_path / "absolute")
        write_random_model(folder, config, seed=8, norm_jitter=0.1, storage=dtype)
        engine = Engine(load_model(folder, dtype, DEVICE), 64 * 6)
        weights = plain_model.read_plain_weights(folder)
        rounding = plain_model.bfloat16_rounding if dtype == "bfloat16" else plain_model.no_rounding
        plain_config = plain_model.PlainConfig(vocab_size=83, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                                               num_key_value_heads=2, head_dim=16, attention_bias=False, rms_norm_eps=1e-6, rope_theta=1.0,
                                               max_position_embeddings=128, tie_word_embeddings=True)
        no_turn = (torch.ones(128, 8), torch.zeros(128, 8))

        def expected(tokens):
            hidden = rounding(plain_model.embedding(weights["model.embed_tokens.weight"], tokens) + weights["model.embed_positions.weight"][: len(tokens)])
            for layer in range(2):
                hidden = plain_model.decoder_block(hidden, weights, f"model.layers.{layer}", plain_config, *no_turn, rounding)
            hidden = plain_model.rms_norm(hidden, weights["model.norm.weight"], 1e-6, rounding)
            return hidden @ weights["model.embed_tokens.weight"].t()

        rng = np.random.default_rng(2)
        requests = [rng.integers(0, 83, size=length).tolist() for length in (90, 33, 7)]
        wanted = [expected(tokens) for tokens in requests]
        slots = [engine.open_sequence() for _ in requests]
        cuts = [70, 20, 3]
        logits = engine.step([StepEntry(slot, tokens[:cut], [0, cut - 1]) for slot, tokens, cut in zip(slots, requests, cuts)]).float().cpu()
        for row, cut in enumerate(cuts):
            assert error(logits[2 * row], wanted[row][0]) < tolerance and error(logits[2 * row + 1], wanted[row][cut - 1]) < tolerance
        for offset in range(4):
            logits = engine.step([StepEntry(slots[i], [requests[i][cuts[i] + offset]], [0]) for i in range(3)]).float().cpu()
            for i in range(3):
                assert error(logits[i], wanted[i][cuts[i] + offset]) < tolerance
        for slot in slots:
            engine.close_sequence(slot)
        engine.cache.check()
        # The positions are felt: a token's logits at position 0 and at position 5 differ although nothing is rotated.
        assert error(wanted[0][0], expected([requests[0][0]] * 6)[5]) > 1e-2
    finally:
        unregister_architecture("ToyAbsoluteForCausalLM")
        unregister("position", "toy_learned_positions")


@pytest.mark.parametrize("dtype,tolerance", [("float32", 1e-4), ("bfloat16", 2e-2)])
def test_windowed_layers_give_pages_back_and_lose_nothing(dtype, tolerance, tmp_path):
    """Every attention layer has a window: a 600-token sequence runs in a cache of 256 positions, pages given back and taken again."""
    from helpers import WINDOW_CONFIG, window_spec, windowed_cache_matches_whole_prompt

    register_architecture("ToyWindowForCausalLM", "toy_window", lambda raw: raw, window_spec)
    try:
        folder = str(tmp_path / "window")
        write_random_model(folder, WINDOW_CONFIG, seed=9, norm_jitter=0.1, storage=dtype)
        windowed_cache_matches_whole_prompt(folder, dtype, DEVICE, tolerance)
    finally:
        unregister_architecture("ToyWindowForCausalLM")
