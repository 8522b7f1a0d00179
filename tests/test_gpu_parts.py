"""Each part alone against the plain implementation, and a toy mixer with state of its own
registered from the test, built and stepped without touching the framework's files."""

import dataclasses
from types import SimpleNamespace

import pytest
import torch

from plain_reference import (
    plain_apply_rope,
    plain_attention,
    plain_config,
    plain_layer,
    plain_layernorm,
    plain_gelu_tanh,
    plain_mlp,
    plain_rope_tables,
)
from tiny_configs import TINY, random_ids, tiny_config, tiny_tensors

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def tol(dtype):
    return dict(atol=2e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)


def make_runtime(dtype, page_size=16):
    from matricxon_b200.parts.base import Runtime

    return Runtime(device=torch.device(DEV), dtype=dtype, page_size=page_size)


def hand_made_context(seq_lens, page_size, pages, start=0):
    """A StepContext for whole sequences starting at ``start``, pages handed out in reverse."""
    from matricxon_b200.engine.step import GroupStep, HostStep, StepContext

    runner = SimpleNamespace(
        status=torch.zeros(1, dtype=torch.int32, device=DEV), sm_count=148, device=torch.device(DEV),
        hidden_buffer=lambda n, h: torch.empty(n, h, device=DEV),
        scratch_buffer=lambda nbytes: torch.empty(nbytes // 4 + 1, device=DEV))
    ctx = StepContext(runner)
    positions, tok_seq, slots, tables = [], [], [], []
    next_page = pages - 1
    width = max((start + n + page_size - 1) // page_size for n in seq_lens)
    for s, n in enumerate(seq_lens):
        table = []
        for _ in range((start + n + page_size - 1) // page_size):
            table.append(next_page)
            next_page -= 1
        assert next_page >= -1
        for i in range(start, start + n):
            positions.append(i)
            tok_seq.append(s)
            slots.append(table[i // page_size] * page_size + i % page_size)
        tables.append(table + [-1] * (width - len(table)))
    as_int = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    ctx.n_tokens, ctx.n_seqs, ctx.max_kv_len = len(positions), len(seq_lens), start + max(seq_lens)
    ctx.positions, ctx.tok_seq = as_int(positions), as_int(tok_seq)
    ctx.groups = [GroupStep(slots=as_int(slots), block_tables=as_int(tables))]
    ctx.host = HostStep(q_lens=list(seq_lens), context_lens=[start] * len(seq_lens),
                        state_slots=list(range(len(seq_lens))), fresh=[True] * len(seq_lens))
    ctx.state_slots = as_int(list(range(len(seq_lens))))
    return ctx


def fetcher(tensors, dtype):
    def fetch(name):
        t = tensors[name]
        want = dtype if t.dim() == 2 else torch.float32
        return t.to(DEV, want).contiguous()

    return fetch


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_mlp_attention_block_alone(name, dtype):
    import matricxon_b200.parts  # noqa: F401  (registers the built-in kinds)
    from matricxon_b200.parts.base import CacheBinding, build_part, part_class

    raw = TINY[name][0]
    cfg = plain_config(raw)
    config = tiny_config(name)
    spec = config.model_spec()
    tensors = tiny_tensors(name, torch.bfloat16 if dtype == torch.bfloat16 else torch.float32)
    plain_w = {k: v.double() for k, v in tensors.items()}
    rt = make_runtime(dtype)
    fetch = fetcher(tensors, dtype)
    seq_lens = [50, 7]
    n = sum(seq_lens)
    torch.manual_seed(3)
    x = torch.randn(n, cfg["hidden"], device=DEV)
    x_cpu = x.double().cpu()
    prefix = "model.layers.1."

    # norm
    norm = build_part("norm", spec.layers[1].mixer_norm, rt, prefix + "input_layernorm.")
    norm.load(fetch)
    h = norm.forward(x)
    h_ref = plain_layernorm(x_cpu, plain_w[prefix + "input_layernorm.weight"],
                            plain_w[prefix + "input_layernorm.bias"], cfg["eps"])
    assert h.dtype == dtype and torch.allclose(h.double().cpu(), h_ref, **tol(dtype))

    # feed-forward: residual + mlp(h)
    mlp = build_part("feed_forward", spec.layers[1].feed_forward, rt, prefix + "mlp.")
    mlp.load(fetch)
    ctx = hand_made_context(seq_lens, 16, 16)
    out = mlp.forward(h, x.clone(), ctx)
    ref = x_cpu + plain_mlp(h.double().cpu(), plain_w, prefix + "mlp.", cfg)
    assert out.dtype == torch.float32 and torch.allclose(out.double().cpu(), ref, **tol(dtype))

    # mixer: residual + attention(h), two whole sequences in one batch
    mixer = build_part("mixer", spec.layers[1].mixer, rt, prefix + "self_attn.")
    mixer.load(fetch)
    kv = torch.full((16, 2, cfg["kv_heads"], 16, cfg["head_dim"]), float("nan"), dtype=dtype, device=DEV)
    binding = CacheBinding(group=0, kv=kv, writes=True)
    out = mixer.forward(h, x.clone(), ctx, binding)
    assert int(ctx.status.item()) == 0
    refs, start = [], 0
    for length in seq_lens:
        piece = h.double().cpu()[start:start + length]
        refs.append(x_cpu[start:start + length] +
                    plain_attention(piece, plain_w, prefix + "self_attn.", cfg, torch.arange(length)))
        start += length
    assert torch.allclose(out.double().cpu(), torch.cat(refs), **tol(dtype))

    # the whole block
    block = part_class("block", spec.layers[1].block)(spec.layers[1], rt, prefix)
    block.load(fetch)
    kv.fill_(float("nan"))
    ctx = hand_made_context(seq_lens, 16, 16)
    out = block.forward(x.clone(), ctx, binding)
    refs, start = [], 0
    for length in seq_lens:
        refs.append(plain_layer(x_cpu[start:start + length], plain_w, 1, cfg, torch.arange(length)))
        start += length
    assert torch.allclose(out.double().cpu(), torch.cat(refs), **tol(dtype))


def test_a_block_leaves_its_last_residual_sum_to_the_next_blocks_norm():
    """With 17 or more rows in bfloat16 the residual products are the library's, and the sum
    ``residual + product + bias`` is formed by the norm that follows (one launch instead of an epilogue
    and a norm). A block returns such a pending sum only to a caller that says it takes one; two blocks
    chained that way give the bits of two blocks run one after the other with the sums added up in between."""
    import matricxon_b200.parts  # noqa: F401
    from matricxon_b200.ops.linear import PendingSum
    from matricxon_b200.parts.base import CacheBinding, part_class

    config = tiny_config("A")
    spec = config.model_spec()
    cfg = plain_config(TINY["A"][0])
    tensors = tiny_tensors("A", torch.bfloat16)
    rt = make_runtime(torch.bfloat16)
    fetch = fetcher(tensors, torch.bfloat16)
    blocks = []
    for layer in (0, 1):
        block = part_class("block", spec.layers[layer].block)(spec.layers[layer], rt, f"model.layers.{layer}.")
        block.load(fetch)
        blocks.append(block)
    seq_lens = [50, 7]
    torch.manual_seed(5)
    x = torch.randn(sum(seq_lens), cfg["hidden"], device=DEV)

    def run(wanted):
        ctx = hand_made_context(seq_lens, 16, 16)
        ctx.pending_sum_wanted = wanted
        stream = x.clone()
        kinds = []
        for block in blocks:
            kv = torch.full((16, 2, cfg["kv_heads"], 16, cfg["head_dim"]), float("nan"), dtype=torch.bfloat16, device=DEV)
            stream = block.forward(stream, ctx, CacheBinding(group=0, kv=kv, writes=True))
            kinds.append(type(stream))
        assert int(ctx.status.item()) == 0
        return (stream.tensor() if isinstance(stream, PendingSum) else stream), kinds

    plain, kinds = run(False)
    assert kinds == [torch.Tensor, torch.Tensor]
    chained, kinds = run(True)
    assert kinds == [PendingSum, PendingSum]
    assert torch.equal(chained, plain)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rotary_part_alone(dtype):
    import matricxon_b200.parts  # noqa: F401
    from matricxon_b200.parts.base import CacheBinding, build_part
    from matricxon_b200.parts.spec import RotarySpec

    heads, kv_heads, dim = 3, 1, 32
    rt = make_runtime(dtype, page_size=8)
    rotary = build_part("position", RotarySpec(rotary_dim=dim, theta=100000.0), rt, "unused.")
    ctx = hand_made_context([11], 8, 32, start=200)
    qkv = torch.randn(11, (heads + 2 * kv_heads) * dim, device=DEV).to(dtype)
    before = qkv.double().cpu()
    kv = torch.zeros(32, 2, kv_heads, 8, dim, dtype=dtype, device=DEV)
    rotary.rotate_and_store(qkv, ctx, CacheBinding(group=0, kv=kv, writes=True), heads, kv_heads, dim)
    cos, sin = plain_rope_tables(torch.arange(200, 211), dim, 100000.0)
    q_ref = plain_apply_rope(before[:, :heads * dim].view(11, heads, dim).transpose(0, 1), cos, sin)
    got = qkv[:, :heads * dim].double().cpu().view(11, heads, dim).transpose(0, 1)
    assert torch.allclose(got, q_ref, **tol(dtype))
    # a reader of someone else's cache stores nothing
    kv.zero_()
    rotary.rotate_and_store(qkv, ctx, CacheBinding(group=0, kv=kv, writes=False), heads, kv_heads, dim)
    assert torch.all(kv == 0)


# --------------------------------------------------------------------------- a toy mixer
def register_toy_parts():
    """A mixer that keeps a running, decayed sum of its projected inputs per request:
    s_t = decay * s_{t-1} + h_t W^T ; out_t = s_t. State of its own, no pages."""
    from matricxon_b200.parts.base import Mixer, StateRequest, register_part
    from matricxon_b200.weights.loader import WeightSpec

    class ToyDecaySpec:
        kind = "toy_decay"

        def __init__(self, hidden_size, decay):
            self.hidden_size, self.decay = hidden_size, decay

    @register_part("mixer", "toy_decay")
    class ToyDecayMixer(Mixer):
        @classmethod
        def weight_specs(cls, spec, prefix):
            return [WeightSpec(prefix + "mix.weight", (spec.hidden_size, spec.hidden_size))]

        @classmethod
        def state_request(cls, spec):
            return StateRequest(shape=(spec.hidden_size,), dtype=torch.float32)

        def load(self, fetch):
            self.weight = fetch(self.prefix + "mix.weight")

        def forward(self, h, residual, ctx, binding):
            projected = (h.float() @ self.weight.float().T)
            out = torch.empty_like(projected)
            start = 0
            for q_len, slot in zip(ctx.host.q_lens, ctx.host.state_slots):
                state = binding.state[slot]
                for i in range(start, start + q_len):           # tokens of a sequence in order
                    state.mul_(self.spec.decay).add_(projected[i])
                    out[i] = state
                start += q_len
            return residual + out

    return ToyDecaySpec


def toy_reference(spec_layers, schedule, weights, cfg, ids, decay):
    """The toy model on the CPU, whole sequence, in double."""
    w = {k: v.double() for k, v in weights.items()}
    x = w["model.embed_tokens.weight"][torch.tensor(ids)]
    positions = torch.arange(len(ids))
    for entry in schedule:
        p = f"model.layers.{entry.layer}."
        h = plain_layernorm(x, w[p + "input_layernorm.weight"], w[p + "input_layernorm.bias"], cfg["eps"])
        if spec_layers[entry.layer].mixer.kind == "toy_decay":
            projected = h @ w[p + "self_attn.mix.weight"].T
            state = torch.zeros(cfg["hidden"], dtype=torch.float64)
            rows = []
            for row in projected:
                state = decay * state + row
                rows.append(state)
            x = x + torch.stack(rows)
        else:
            x = x + plain_attention(h, w, p + "self_attn.", cfg, positions)
        h = plain_layernorm(x, w[p + "post_attention_layernorm.weight"],
                            w[p + "post_attention_layernorm.bias"], cfg["eps"])
        x = x + plain_mlp(h, w, p + "mlp.", cfg)
    x = plain_layernorm(x, w["model.norm.weight"], w["model.norm.bias"], cfg["eps"])
    return x @ w["model.embed_tokens.weight"].T


def test_toy_mixer_with_state_is_registered_built_and_stepped():
    """Layers of different kinds in one model, a layer named twice in the schedule (weights
    shared, caches and states apart), and per-request state carried across steps."""
    import matricxon_b200.parts  # noqa: F401
    from matricxon_b200.engine.core import EngineCore
    from matricxon_b200.engine.step import StepEntry
    from matricxon_b200.models.decoder import DecoderModel, model_weight_specs
    from matricxon_b200.parts.spec import LayerSpec, ModelSpec, ScheduleEntry
    from matricxon_b200.weights.loader import DictSource, make_fetcher
    from matricxon_b200.weights.random_init import RandomInit, RandomSource

    ToyDecaySpec = register_toy_parts()
    base = tiny_config("A").model_spec()
    attention_layer = base.layers[0]
    toy_layer = dataclasses.replace(attention_layer, mixer=ToyDecaySpec(base.hidden_size, 0.5))
    schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1))
    spec = dataclasses.replace(base, layers=(attention_layer, toy_layer), schedule=schedule)
    specs = model_weight_specs(spec)
    assert any(s.name == "model.layers.1.self_attn.mix.weight" for s in specs)
    source = RandomSource(specs, seed=11, init=RandomInit(0.05, 0.02, 0.02, 0.02))
    weights = {name: source.read(name) for name in source.names()}

    rt = make_runtime(torch.float32)
    model = DecoderModel(spec, rt)
    assert model.cache_plan.state_bytes_per_request == 2 * 64 * 4       # two executions of the toy layer
    assert model.cache_plan.groups[0].entries == (0, 2)                 # two caches for attention layer 0
    model.load(make_fetcher(specs, DictSource(weights), torch.float32, DEV))
    core = EngineCore(model, max_cache_tokens=256, max_requests=4)

    cfg = plain_config(TINY["A"][0])
    prompts = {"x": random_ids(45, 512, 1), "y": random_ids(20, 512, 2)}
    refs = {k: toy_reference(spec.layers, schedule, weights, cfg, ids, 0.5) for k, ids in prompts.items()}
    for rid in prompts:
        core.cache.add_request(rid)
    got = {rid: [] for rid in prompts}
    done = {rid: 0 for rid in prompts}
    sizes = [5, 1, 9, 2, 1, 1, 13, 3]
    turn = 0
    while any(done[r] < len(prompts[r]) for r in prompts):
        entries = []
        for rid, ids in prompts.items():
            if done[rid] < len(ids):
                size = min(sizes[turn % len(sizes)], len(ids) - done[rid])
                turn += 1
                entries.append(StepEntry(rid, ids[done[rid]:done[rid] + size], list(range(size))))
                done[rid] += size
        logits = core.runner.run(entries).cpu()
        core.runner.check_status()
        row = 0
        for entry in entries:
            got[entry.request_id].append(logits[row:row + len(entry.tokens)])
            row += len(entry.tokens)
    for rid in prompts:
        assert torch.allclose(torch.cat(got[rid]).double(), refs[rid], atol=5e-5), rid
    # a slot given to a new request starts from zero again
    core.cache.free_request("x")
    core.cache.add_request("z")
    logits = core.runner.run([StepEntry("z", prompts["x"], list(range(45)))]).cpu()
    assert torch.allclose(logits.double(), refs["x"], atol=5e-5)


# ------------------------------------------- a toy position encoding and a toy routed feed-forward
def register_toy_position_and_router():
    """Two more kinds registered from the test file alone.

    ``toy_distance_decay`` (a position encoding): q is scaled by a^p and k by a^-p at position p,
    so the score of (p, j) carries the factor a^(p - j); then k and v are stored as they are.
    ``toy_top1_experts`` (a feed-forward): router logits and their softmax in float; the token goes
    through the one expert with the largest probability (an ungated tanh-GELU MLP) and the
    result is scaled by that probability."""
    from matricxon_b200.parts.base import FeedForward, PositionEncoding, register_part
    from matricxon_b200.parts.rotary import store_without_rotation
    from matricxon_b200.weights.loader import WeightSpec

    class ToyDecaySpec:
        kind = "toy_distance_decay"

        def __init__(self, base):
            self.base = base

    class ToyExpertsSpec:
        kind = "toy_top1_experts"

        def __init__(self, hidden_size, intermediate_size, experts):
            self.hidden_size, self.intermediate_size, self.experts = hidden_size, intermediate_size, experts

    @register_part("position", "toy_distance_decay")
    class ToyDistanceDecay(PositionEncoding):
        def rotate_and_store(self, qkv, ctx, binding, n_heads, n_kv_heads, head_dim):
            factor = (self.spec.base ** ctx.positions.double()).float()[:, None]
            q_cols, k_cols = n_heads * head_dim, n_kv_heads * head_dim
            qkv[:, :q_cols] = (qkv[:, :q_cols].float() * factor).to(qkv.dtype)
            qkv[:, q_cols:q_cols + k_cols] = (qkv[:, q_cols:q_cols + k_cols].float() / factor).to(qkv.dtype)
            store_without_rotation(qkv, ctx, binding, n_heads, n_kv_heads, head_dim, self.runtime.page_size)

    @register_part("feed_forward", "toy_top1_experts")
    class ToyTop1Experts(FeedForward):
        @classmethod
        def weight_specs(cls, spec, prefix):
            specs = [WeightSpec(prefix + "router.weight", (spec.experts, spec.hidden_size))]
            for e in range(spec.experts):
                specs.append(WeightSpec(f"{prefix}experts.{e}.up.weight", (spec.intermediate_size, spec.hidden_size)))
                specs.append(WeightSpec(f"{prefix}experts.{e}.down.weight", (spec.hidden_size, spec.intermediate_size)))
            return specs

        def load(self, fetch):
            self.router = fetch(self.prefix + "router.weight")
            self.up = [fetch(f"{self.prefix}experts.{e}.up.weight") for e in range(self.spec.experts)]
            self.down = [fetch(f"{self.prefix}experts.{e}.down.weight") for e in range(self.spec.experts)]

        def forward(self, h, residual, ctx):
            probs = torch.softmax(h.float() @ self.router.float().T, dim=-1)
            weight, choice = probs.max(dim=-1)
            out = torch.zeros_like(residual)
            for e in range(self.spec.experts):
                rows = torch.nonzero(choice == e).flatten()
                if rows.numel():
                    mid = torch.nn.functional.gelu(h[rows].float() @ self.up[e].float().T, approximate="tanh")
                    out[rows] = (mid @ self.down[e].float().T) * weight[rows, None]
            return residual + out

    return ToyDecaySpec, ToyExpertsSpec


def test_toy_position_encoding_and_routed_feed_forward_beside_the_stock_parts():
    """A layer whose attention uses a position encoding defined here and whose feed-forward routes
    tokens between experts, beside a stock StarCoder2 layer, built from specs and stepped in
    portions for two requests: nothing in the package names these kinds."""
    import dataclasses

    import matricxon_b200.parts  # noqa: F401
    from matricxon_b200.engine.core import EngineCore
    from matricxon_b200.engine.step import StepEntry
    from matricxon_b200.models.decoder import DecoderModel, model_weight_specs
    from matricxon_b200.parts.spec import LayerSpec, ModelSpec, ScheduleEntry
    from matricxon_b200.weights.loader import DictSource, make_fetcher
    from matricxon_b200.weights.random_init import RandomInit, RandomSource
    from plain_reference import plain_attention_core, plain_linear

    ToyDecaySpec, ToyExpertsSpec = register_toy_position_and_router()
    base = tiny_config("A").model_spec()
    stock = base.layers[0]
    decay_base, experts, inter = 1.01, 3, 80
    toy_attention = dataclasses.replace(stock.mixer, position=ToyDecaySpec(decay_base))
    toy_layer = dataclasses.replace(stock, mixer=toy_attention,
                                    feed_forward=ToyExpertsSpec(base.hidden_size, inter, experts))
    schedule = (ScheduleEntry(0), ScheduleEntry(1))
    spec = dataclasses.replace(base, layers=(toy_layer, stock), schedule=schedule)
    specs = model_weight_specs(spec)
    assert any(s.name == "model.layers.0.mlp.experts.2.down.weight" for s in specs)
    source = RandomSource(specs, seed=5, init=RandomInit(0.08, 0.02, 0.02, 0.02))
    weights = {name: source.read(name) for name in source.names()}
    model = DecoderModel(spec, make_runtime(torch.float32))
    assert len(model.cache_plan.groups) == 1            # same geometry and window: one group of pages
    model.load(make_fetcher(specs, DictSource(weights), torch.float32, DEV))
    core = EngineCore(model, max_cache_tokens=256, max_requests=4)
    cfg = plain_config(TINY["A"][0])

    def reference(ids):
        w = {k: v.double() for k, v in weights.items()}
        t = len(ids)
        heads, kv_heads, d = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
        positions = torch.arange(t)
        x = w["model.embed_tokens.weight"][torch.tensor(ids)]
        # layer 0: toy position encoding, toy experts
        p = "model.layers.0."
        h = plain_layernorm(x, w[p + "input_layernorm.weight"], w[p + "input_layernorm.bias"], cfg["eps"])
        q = plain_linear(h, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.q_proj.bias"]).view(t, heads, d)
        k = plain_linear(h, w[p + "self_attn.k_proj.weight"], w[p + "self_attn.k_proj.bias"]).view(t, kv_heads, d)
        v = plain_linear(h, w[p + "self_attn.v_proj.weight"], w[p + "self_attn.v_proj.bias"]).view(t, kv_heads, d)
        factor = (decay_base ** positions.double())[:, None, None]
        o = plain_attention_core((q * factor).transpose(0, 1), (k / factor).transpose(0, 1), v.transpose(0, 1),
                                 d ** -0.5, cfg["window"])
        x = x + plain_linear(o.transpose(0, 1).reshape(t, heads * d), w[p + "self_attn.o_proj.weight"],
                             w[p + "self_attn.o_proj.bias"])
        h = plain_layernorm(x, w[p + "post_attention_layernorm.weight"], w[p + "post_attention_layernorm.bias"],
                            cfg["eps"])
        probs = torch.softmax(h @ w[p + "mlp.router.weight"].T, dim=-1)
        gate, choice = probs.max(dim=-1)
        rows = []
        for i in range(t):
            e = int(choice[i])
            mid = plain_gelu_tanh(h[i] @ w[f"{p}mlp.experts.{e}.up.weight"].T)
            rows.append((mid @ w[f"{p}mlp.experts.{e}.down.weight"].T) * gate[i])
        x = x + torch.stack(rows)
        # layer 1: the stock layer
        p = "model.layers.1."
        h = plain_layernorm(x, w[p + "input_layernorm.weight"], w[p + "input_layernorm.bias"], cfg["eps"])
        x = x + plain_attention(h, w, p + "self_attn.", cfg, positions)
        h = plain_layernorm(x, w[p + "post_attention_layernorm.weight"], w[p + "post_attention_layernorm.bias"],
                            cfg["eps"])
        x = x + plain_mlp(h, w, p + "mlp.", cfg)
        x = plain_layernorm(x, w["model.norm.weight"], w["model.norm.bias"], cfg["eps"])
        return x @ w["model.embed_tokens.weight"].T

    prompts = {"x": random_ids(50, 512, 3), "y": random_ids(23, 512, 4)}
    refs = {rid: reference(ids) for rid, ids in prompts.items()}
    for rid in prompts:
        core.cache.add_request(rid)
    got = {rid: [] for rid in prompts}
    done = {rid: 0 for rid in prompts}
    sizes = [7, 1, 2, 11, 1, 1, 5, 3]
    turn = 0
    while any(done[r] < len(prompts[r]) for r in prompts):
        entries = []
        for rid, ids in prompts.items():
            if done[rid] < len(ids):
                size = min(sizes[turn % len(sizes)], len(ids) - done[rid])
                turn += 1
                entries.append(StepEntry(rid, ids[done[rid]:done[rid] + size], list(range(size))))
                done[rid] += size
        logits = core.runner.run(entries).cpu()
        core.runner.check_status()
        row = 0
        for entry in entries:
            got[entry.request_id].append(logits[row:row + len(entry.tokens)])
            row += len(entry.tokens)
    for rid in prompts:
        worst = (torch.cat(got[rid]).double() - refs[rid]).abs().max()
        assert torch.allclose(torch.cat(got[rid]).double(), refs[rid], atol=1e-4), (rid, float(worst))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_with_a_fused_differently_named_qkv_tensor(dtype):
    """A checkpoint that stores q, k and v as one tensor under other names is a matter of the
    spec's name fields: the part is the stock one, nothing in the package changes, and the logits
    equal the stock model's on the same numbers."""
    from matricxon_b200.engine.core import EngineCore
    from matricxon_b200.engine.step import StepEntry
    from matricxon_b200.models.decoder import DecoderModel, model_weight_specs
    from matricxon_b200.weights.loader import DictSource, make_fetcher

    base = tiny_config("A").model_spec()
    stock_layer = base.layers[0]
    fused_mixer = dataclasses.replace(stock_layer.mixer, projection_names=("c_attn",), output_name="dense")
    fused_layer = dataclasses.replace(stock_layer, mixer=fused_mixer, mixer_name="attn",
                                      mixer_norm_name="ln_1", ffn_norm_name="ln_2")
    spec = dataclasses.replace(base, layers=(fused_layer,) * len(base.layers), embedding_name="wte",
                               layer_prefix="h", final_norm_name="ln_f")
    names = {s.name for s in model_weight_specs(spec)}
    assert "h.0.attn.c_attn.weight" in names and "h.1.attn.dense.bias" in names and "wte.weight" in names
    assert not any("q_proj" in name or "model." in name for name in names)

    stock = tiny_tensors("A", dtype)
    renamed = {}
    for layer in range(len(base.layers)):
        old, new = f"model.layers.{layer}.", f"h.{layer}."
        for kind in ("weight", "bias"):
            renamed[f"{new}attn.c_attn.{kind}"] = torch.cat(
                [stock[f"{old}self_attn.{n}.{kind}"] for n in ("q_proj", "k_proj", "v_proj")])
            renamed[f"{new}attn.dense.{kind}"] = stock[f"{old}self_attn.o_proj.{kind}"]
            renamed[f"{new}ln_1.{kind}"] = stock[f"{old}input_layernorm.{kind}"]
            renamed[f"{new}ln_2.{kind}"] = stock[f"{old}post_attention_layernorm.{kind}"]
            for n in ("c_fc", "c_proj"):
                renamed[f"{new}mlp.{n}.{kind}"] = stock[f"{old}mlp.{n}.{kind}"]
    renamed["wte.weight"] = stock["model.embed_tokens.weight"]
    renamed["ln_f.weight"], renamed["ln_f.bias"] = stock["model.norm.weight"], stock["model.norm.bias"]
    assert set(renamed) == names

    ids = random_ids(45, TINY["A"][0]["vocab_size"], seed=4)
    outputs = []
    for model_spec, tensors in ((base, stock), (spec, renamed)):
        model = DecoderModel(model_spec, make_runtime(dtype))
        model.load(make_fetcher(model_weight_specs(model_spec), DictSource(tensors), dtype, DEV))
        core = EngineCore(model, max_cache_tokens=128, max_requests=2)
        core.cache.add_request("r")
        first = core.runner.run([StepEntry("r", ids[:30], list(range(30)))]).clone()
        rest = core.runner.run([StepEntry("r", ids[30:], list(range(15)))]).clone()
        core.runner.check_status()
        outputs.append(torch.cat([first, rest]))
    assert torch.equal(outputs[0], outputs[1])


# ------------------------------------------- a toy mixer whose paged cache is not a key/value pair
def test_toy_mixer_with_a_one_plane_windowed_cache():
    """``toy_latent_mean``: every token stores ONE projected vector in the paged cache (one plane,
    one "head" as wide as the vector) and outputs the mean of the vectors of the last ``window``
    positions, itself included. Its pages live in a pool of their own beside the attention
    layers' (another geometry, another window), are written through the step's slots, read through
    its block tables, and are given back as the window passes them. Defined here, registered
    here; the package does not know it."""
    from matricxon_b200.engine.core import EngineCore
    from matricxon_b200.engine.step import StepEntry
    from matricxon_b200.models.decoder import DecoderModel, model_weight_specs
    from matricxon_b200.parts.base import KVCacheRequest, Mixer, register_part
    from matricxon_b200.parts.spec import ScheduleEntry
    from matricxon_b200.weights.loader import DictSource, WeightSpec, make_fetcher
    from matricxon_b200.weights.random_init import RandomInit, RandomSource

    class ToyLatentSpec:
        kind = "toy_latent_mean"

        def __init__(self, hidden_size, latent, window):
            self.hidden_size, self.latent, self.window = hidden_size, latent, window

    @register_part("mixer", "toy_latent_mean")
    class ToyLatentMean(Mixer):
        @classmethod
        def weight_specs(cls, spec, prefix):
            return [WeightSpec(prefix + "down.weight", (spec.latent, spec.hidden_size)),
                    WeightSpec(prefix + "up.weight", (spec.hidden_size, spec.latent))]

        @classmethod
        def cache_request(cls, spec):
            return KVCacheRequest(num_kv_heads=1, head_dim=spec.latent, window=spec.window, planes=1)

        def load(self, fetch):
            self.down, self.up = fetch(self.prefix + "down.weight"), fetch(self.prefix + "up.weight")

        def forward(self, h, residual, ctx, binding):
            pages, planes, heads, page_size, latent = binding.kv.shape
            assert (planes, heads, latent) == (1, 1, self.spec.latent)
            flat = binding.kv.view(pages * page_size, latent)          # slot -> vector
            group = ctx.groups[binding.group]
            vectors = h.float() @ self.down.float().T
            if binding.writes:
                flat[group.slots.long()] = vectors.to(flat.dtype)
            tables = group.block_tables.cpu()
            out = torch.empty_like(vectors)
            row = 0
            for seq, (q_len, start) in enumerate(zip(ctx.host.q_lens, ctx.host.context_lens)):
                for position in range(start, start + q_len):
                    seen = range(max(0, position - self.spec.window + 1), position + 1)
                    slots = [int(tables[seq, j // page_size]) * page_size + j % page_size for j in seen]
                    assert min(slots) >= 0, "a position inside the window has lost its page"
                    out[row] = flat[torch.tensor(slots, device=h.device)].float().mean(dim=0)
                    row += 1
            return residual + out @ self.up.float().T

    base = tiny_config("A").model_spec()
    window, latent = 9, 48
    toy_layer = dataclasses.replace(base.layers[0], mixer=ToyLatentSpec(base.hidden_size, latent, window))
    schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1))
    spec = dataclasses.replace(base, layers=(base.layers[0], toy_layer), schedule=schedule)
    specs = model_weight_specs(spec)
    source = RandomSource(specs, seed=3, init=RandomInit(0.05, 0.02, 0.02, 0.02))
    weights = {name: source.read(name) for name in source.names()}
    model = DecoderModel(spec, make_runtime(torch.float32))
    plan = model.cache_plan
    assert len(plan.groups) == 2 and plan.groups[1].entries == (1, 2)       # the toy layer runs twice
    assert plan.groups[1].request == KVCacheRequest(1, latent, window, planes=1)
    model.load(make_fetcher(specs, DictSource(weights), torch.float32, DEV))
    core = EngineCore(model, max_cache_tokens=128, max_requests=2, poison_cache=True)
    assert tuple(core.storage.groups[1].shape) == (2, 8, 1, 1, 16, latent)

    cfg = plain_config(TINY["A"][0])
    ids = random_ids(60, 512, 9)

    def reference():
        w = {k: v.double() for k, v in weights.items()}
        x = w["model.embed_tokens.weight"][torch.tensor(ids)]
        positions = torch.arange(len(ids))
        for entry in schedule:
            p = f"model.layers.{entry.layer}."
            hidden = plain_layernorm(x, w[p + "input_layernorm.weight"], w[p + "input_layernorm.bias"], cfg["eps"])
            if entry.layer == 1:
                vectors = hidden @ w[p + "self_attn.down.weight"].T
                means = torch.stack([vectors[max(0, t - window + 1):t + 1].mean(dim=0) for t in range(len(ids))])
                x = x + means @ w[p + "self_attn.up.weight"].T
            else:
                x = x + plain_attention(hidden, w, p + "self_attn.", cfg, positions)
            hidden = plain_layernorm(x, w[p + "post_attention_layernorm.weight"],
                                     w[p + "post_attention_layernorm.bias"], cfg["eps"])
            x = x + plain_mlp(hidden, w, p + "mlp.", cfg)
        x = plain_layernorm(x, w["model.norm.weight"], w["model.norm.bias"], cfg["eps"])
        return x @ w["model.embed_tokens.weight"].T

    expected = reference()
    core.cache.add_request("r")
    got, done = [], 0
    for size in [7, 2, 16, 1, 1, 5, 11, 3, 1, 13]:
        size = min(size, len(ids) - done)
        if size == 0:
            break
        got.append(core.runner.run([StepEntry("r", ids[done:done + size], list(range(size)))]).cpu())
        core.runner.check_status()
        done += size
        core.cache.check_invariants()
    assert done == len(ids)
    assert torch.allclose(torch.cat(got).double(), expected, atol=5e-5)
    # the toy group's window of 9 keeps at most two pages of 16; the attention group's window of 32 three
    assert len(core.cache.held_pages("r", 1)) <= 2 and len(core.cache.held_pages("r", 0)) <= 3
    assert core.cache.pages_reused > 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_scale_head_bias_and_logit_cap_are_spec_fields(dtype):
    """What some architectures do around the layers is data of the model's description too: the
    embeddings times a constant, a bias on the head, scores squashed to cap * tanh(score / cap).
    A stock tiny model with the three switched on, against the plain parts."""
    from matricxon_b200.engine.core import EngineCore
    from matricxon_b200.engine.step import StepEntry
    from matricxon_b200.models.decoder import DecoderModel, model_weight_specs
    from matricxon_b200.weights.loader import DictSource, make_fetcher
    from plain_reference import plain_embedding, plain_layer

    scale, cap = 1.75, 0.6
    base = tiny_config("A").model_spec()
    spec = dataclasses.replace(base, embedding_scale=scale, head_bias=True, logit_softcap=cap)
    names = {s.name for s in model_weight_specs(spec)}
    assert "lm_head.bias" in names
    tensors = dict(tiny_tensors("A", dtype))
    torch.manual_seed(3)
    tensors["lm_head.bias"] = torch.randn(TINY["A"][0]["vocab_size"]) * 0.3
    model = DecoderModel(spec, make_runtime(dtype))
    model.load(make_fetcher(model_weight_specs(spec), DictSource(tensors), dtype, DEV))
    core = EngineCore(model, max_cache_tokens=128, max_requests=2)
    ids = random_ids(40, TINY["A"][0]["vocab_size"], seed=8)
    core.cache.add_request("r")
    got = torch.cat([core.runner.run([StepEntry("r", ids[:25], list(range(25)))]).clone(),
                     core.runner.run([StepEntry("r", ids[25:], list(range(15)))]).clone()]).double().cpu()
    core.runner.check_status()

    cfg = plain_config(TINY["A"][0])
    w = {k: v.double() for k, v in tensors.items()}
    x = plain_embedding(torch.tensor(ids), w["model.embed_tokens.weight"]) * scale
    for layer in range(cfg["layers"]):
        x = plain_layer(x, w, layer, cfg, torch.arange(len(ids)))
    x = plain_layernorm(x, w["model.norm.weight"], w["model.norm.bias"], cfg["eps"])
    scores = x @ w["model.embed_tokens.weight"].T + w["lm_head.bias"]
    expected = cap * torch.tanh(scores / cap)
    assert float(expected.abs().max()) > 0.5 * cap          # the cap bites
    assert torch.allclose(got, expected, **(dict(atol=2e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)))
