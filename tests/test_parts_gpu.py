"""Each part alone against its plain statement, at sizes other than the tiny models', and the
generality of the assembly: a toy architecture, defined here and registered without touching
the package, with a mixer that keeps a state of its own, a layer that runs twice and a run
that reads another run's cache; stepped in every cutting against a plain whole-sequence
computation written here."""

from __future__ import annotations

import json
from dataclasses import dataclass
from types import SimpleNamespace

import pytest
import torch

import helpers
import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, scale=1.0):
    return dict(atol=(3e-5 if dtype == torch.float32 else 3e-2) * scale, rtol=3e-5 if dtype == torch.float32 else 3e-2)


def rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).cuda()


# --------------------------------------------------------------------------- a harness for one part


class Harness:
    """A cache manager, device pools and a context builder around a single part."""

    def __init__(self, needs, dtype, page_size=4, num_pages=64, max_seqs=4, vocab=50, max_len=512):
        import miniserve_b200  # noqa: F401
        from miniserve_b200.cache import CacheManager
        from miniserve_b200.cache.storage import CacheStorage
        from miniserve_b200.engine.step import StepFunction
        from miniserve_b200.parts import CacheGroup

        groups = [CacheGroup(need, 1) for need in needs]
        self.manager = CacheManager(groups, page_size, num_pages, max_seqs)
        self.storage = CacheStorage(groups, page_size, num_pages, max_seqs, dtype, torch.device("cuda"))
        model = SimpleNamespace(device=torch.device("cuda"), dtype=dtype, spec=SimpleNamespace(vocab_size=vocab))
        self.step_function = StepFunction(model, self.storage, self.manager, max_len)

    def context(self, portions):
        """``portions``: {request id: number of new tokens}; admits unknown ids."""
        from miniserve_b200.engine.step import StepEntry

        for rid in portions:
            if rid not in self.manager.requests:
                entry = self.manager.admit(rid)
                self.storage.reset_slot(entry.slot, 0.0, 1.0, 0, 0)
        reservation = self.manager.prepare(list(portions.items()))
        ctx = self.step_function.build_context([StepEntry(rid, [0] * n, []) for rid, n in portions.items()], reservation)
        self.manager.commit(reservation)
        return ctx

    def view(self, ctx, group=0):
        from miniserve_b200.parts import RunCache
        return self.storage.run_view(RunCache(group, 0, True), ctx)


# --------------------------------------------------------------------------- parts alone


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("size,eps", [(40, 1e-5), (136, 1e-6), (3000, 1e-3)])
def test_norm_part(dtype, size, eps):
    from miniserve_b200.parts import NORMS, PartSpec

    part = NORMS.build(PartSpec("rms", dict(name="w", size=size, eps=eps)), prefix="layer.")
    assert [(s.name, s.shape, s.kind) for s in part.param_specs()] == [("layer.w", (size,), "vector")]
    weight = (1 + rand((size,), torch.float32, 1, 0.2)).to(dtype)
    part.load({"layer.w": weight})
    residual, delta = rand((5, size), torch.float32, 2, 2.0), rand((5, size), dtype, 3)
    expected_sum = residual.double() + delta.double()
    out = torch.empty((5, size), dtype=dtype).cuda()
    part.add_and_norm(residual, delta, out)
    expected = plain.plain_rmsnorm(expected_sum, weight.double(), eps)
    assert torch.allclose(residual.double(), expected_sum, atol=1e-6)
    assert torch.allclose(out.double(), expected, **tol(dtype, 3.0))


@pytest.mark.parametrize("head_dim,rotary_dim,interleaved,theta", [(64, None, False, 1e4), (48, 32, False, 5e5), (32, 32, True, 1e6), (128, 64, True, 1e4)])
def test_position_part_inside_the_attention_kernel(head_dim, rotary_dim, interleaved, theta):
    """The rotation tables and their use by the fused kernel, against a direct statement of the rotation."""
    from miniserve_b200 import kernels
    from miniserve_b200.parts import POSITIONS, PartSpec

    part = POSITIONS.build(PartSpec("rope", dict(head_dim=head_dim, theta=theta, rotary_dim=rotary_dim, interleaved=interleaved)))
    positions = torch.tensor([0, 1, 5, 300, 4095], dtype=torch.int32).cuda()
    ctx = SimpleNamespace(n_tokens=5, positions=positions, device=torch.device("cuda"), memo={})
    table, rot, inter = part.fused_args(ctx)
    assert part.fused_args(ctx)[0] is table                      # computed once per step
    n_q, n_kv = 3, 1
    qkv = rand((5, (n_q + 2 * n_kv) * head_dim), torch.float32, 4)
    pool_k = torch.zeros((2, n_kv, 4, head_dim), dtype=torch.float32).cuda()
    pool_v = torch.zeros_like(pool_k)
    q_out = torch.empty((5, n_q, head_dim), dtype=torch.float32).cuda()
    slots = torch.arange(5, dtype=torch.int32).cuda()
    kernels.qk_norm_rope_append(qkv, slots, None, None, 1e-6, table, rot, inter, pool_k, pool_v, n_q, n_kv, head_dim, q_out)
    heads = qkv.view(5, n_q + 2 * n_kv, head_dim).double().cpu()
    inv_freq = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    angles = (positions.cpu().float()[:, None] * inv_freq[None, :]).double()
    cos, sin = angles.cos()[:, None, :], angles.sin()[:, None, :]
    expected = heads[:, :n_q].clone()
    x = heads[:, :n_q]
    if interleaved:
        a, b = x[..., 0:rot:2], x[..., 1:rot:2]
        expected[..., 0:rot:2], expected[..., 1:rot:2] = a * cos - b * sin, b * cos + a * sin
    else:
        a, b = x[..., :rot // 2], x[..., rot // 2:rot]
        expected[..., :rot // 2], expected[..., rot // 2:rot] = a * cos - b * sin, b * cos + a * sin
    assert torch.allclose(q_out.double().cpu(), expected, atol=2e-5)


def attention_weights(hidden, n_q, n_kv, d, dtype, seed, qk_norm=True):
    w = {"a.q_proj.weight": rand((n_q * d, hidden), dtype, seed, 0.08), "a.k_proj.weight": rand((n_kv * d, hidden), dtype, seed + 1, 0.08),
         "a.v_proj.weight": rand((n_kv * d, hidden), dtype, seed + 2, 0.08), "a.o_proj.weight": rand((hidden, n_q * d), dtype, seed + 3, 0.08)}
    if qk_norm:
        w["a.q_norm.weight"] = (1 + rand((d,), torch.float32, seed + 4, 0.1)).to(dtype)
        w["a.k_norm.weight"] = (1 + rand((d,), torch.float32, seed + 5, 0.1)).to(dtype)
    return w


def plain_attention_part(x, w, n_q, n_kv, d, eps, theta, positions, window, qk_norm=True, scale=None):
    n = x.shape[0]
    q = (x @ w["a.q_proj.weight"].double().T).view(n, n_q, d)
    k = (x @ w["a.k_proj.weight"].double().T).view(n, n_kv, d)
    v = (x @ w["a.v_proj.weight"].double().T).view(n, n_kv, d)
    if qk_norm:
        q = plain.plain_rmsnorm(q, w["a.q_norm.weight"].double(), eps)
        k = plain.plain_rmsnorm(k, w["a.k_norm.weight"].double(), eps)
    cos, sin = plain.plain_rope_tables(positions, d, theta, torch.float64)
    q, k = plain.plain_apply_rope(q, cos, sin), plain.plain_apply_rope(k, cos, sin)
    if scale is not None:
        q = q * (scale / d ** -0.5)
    return plain.plain_attention(q, k, v, positions, window).reshape(n, n_q * d) @ w["a.o_proj.weight"].double().T


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,n_q,n_kv,d,window,qk_norm,scale", [
    (80, 5, 1, 32, None, True, None), (104, 4, 4, 64, 9, False, None), (56, 6, 2, 16, None, True, 0.3), (72, 2, 1, 128, 17, True, None)])
def test_attention_part_in_portions(dtype, hidden, n_q, n_kv, d, window, qk_norm, scale):
    """The mixer alone: a sequence fed in three portions (the cache carries what came before)."""
    from miniserve_b200.parts import MIXERS, PagedKVNeed, PartSpec

    spec = PartSpec("attention", dict(hidden_size=hidden, num_heads=n_q, num_kv_heads=n_kv, head_dim=d, qk_norm=qk_norm, eps=1e-5,
                                      position=PartSpec("rope", dict(theta=3e4)), window=window, scale=scale))
    part = MIXERS.build(spec, prefix="a.")
    assert part.cache_need() == PagedKVNeed(n_kv, d, window)
    w = attention_weights(hidden, n_q, n_kv, d, dtype, 10, qk_norm)
    assert sorted(s.name for s in part.param_specs()) == sorted(w)
    part.load(w)
    harness = Harness([part.cache_need()], dtype, page_size=4)
    total = 41
    x = rand((total, hidden), dtype, 20)
    got = []
    for start, end in ((0, 13), (13, 14), (14, 41)):
        ctx = harness.context({"r": end - start})
        got.append(part.forward(x[start:end].contiguous(), ctx, harness.view(ctx)))
    expected = plain_attention_part(x.double().cpu(), {k: v.cpu() for k, v in w.items()}, n_q, n_kv, d, 1e-5, 3e4,
                                    torch.arange(total), window, qk_norm, scale)
    assert torch.allclose(torch.cat(got).double().cpu(), expected, **tol(dtype, float(expected.abs().max())))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,inter,rows", [(72, 200, 5), (96, 40, 70), (136, 264, 1), (88, 100, 4)])
def test_feed_forward_part(dtype, hidden, inter, rows):
    from miniserve_b200.parts import FEED_FORWARDS, PartSpec

    part = FEED_FORWARDS.build(PartSpec("gated_mlp", dict(hidden_size=hidden, intermediate_size=inter)), prefix="m.")
    w = {"m.gate_proj.weight": rand((inter, hidden), dtype, 30, 0.1), "m.up_proj.weight": rand((inter, hidden), dtype, 31, 0.1),
         "m.down_proj.weight": rand((hidden, inter), dtype, 32, 0.1)}
    assert sorted(s.name for s in part.param_specs()) == sorted(w)
    part.load(w)
    x = rand((rows, hidden), dtype, 33)
    from miniserve_b200.parts import PagedKVNeed
    out = part.forward(x, Harness([PagedKVNeed(1, 16, None)], dtype, num_pages=32).context({"a": rows}))
    expected = plain.plain_swiglu(x.double(), *(w[k].double() for k in ("m.gate_proj.weight", "m.up_proj.weight", "m.down_proj.weight")))
    assert torch.allclose(out.double(), expected, **tol(dtype, float(expected.abs().max())))


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_part(dtype):
    """The pre-norm arrangement alone: pending delta in, pending delta out, residual updated in place."""
    from miniserve_b200.parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, PartSpec

    hidden, n_q, n_kv, d, inter, eps = 88, 4, 2, 32, 120, 1e-6
    mixer = MIXERS.build(PartSpec("attention", dict(hidden_size=hidden, num_heads=n_q, num_kv_heads=n_kv, head_dim=d, qk_norm=True,
                                                    eps=eps, position=PartSpec("rope", dict(theta=1e4)))), prefix="a.")
    ffn = FEED_FORWARDS.build(PartSpec("gated_mlp", dict(hidden_size=hidden, intermediate_size=inter)), prefix="m.")
    norm1 = NORMS.build(PartSpec("rms", dict(name="n1", size=hidden, eps=eps)), prefix="")
    norm2 = NORMS.build(PartSpec("rms", dict(name="n2", size=hidden, eps=eps)), prefix="")
    block = BLOCKS.build(PartSpec("pre_norm"), mixer=mixer, feed_forward=ffn, mixer_norm=norm1, feed_forward_norm=norm2)
    w = attention_weights(hidden, n_q, n_kv, d, dtype, 40)
    w.update({"m.gate_proj.weight": rand((inter, hidden), dtype, 46, 0.1), "m.up_proj.weight": rand((inter, hidden), dtype, 47, 0.1),
              "m.down_proj.weight": rand((hidden, inter), dtype, 48, 0.1),
              "n1": (1 + rand((hidden,), torch.float32, 49, 0.1)).to(dtype), "n2": (1 + rand((hidden,), torch.float32, 50, 0.1)).to(dtype)})
    for part in block.parts():
        part.load({s.name: w[s.name] for s in part.param_specs()})
    harness = Harness([mixer.cache_need()], dtype)
    n = 19
    residual, pending = rand((n, hidden), torch.float32, 51), rand((n, hidden), dtype, 52)
    ctx = harness.context({"r": n})
    ctx.dtype = dtype
    h0 = residual.double().cpu() + pending.double().cpu()
    delta = block.forward(residual, pending, ctx, harness.view(ctx))
    wd = {k: v.double().cpu() for k, v in w.items()}
    h1 = h0 + plain_attention_part(plain.plain_rmsnorm(h0, wd["n1"], eps), wd, n_q, n_kv, d, eps, 1e4, torch.arange(n), None)
    expected_delta = plain.plain_swiglu(plain.plain_rmsnorm(h1, wd["n2"], eps), wd["m.gate_proj.weight"], wd["m.up_proj.weight"],
                                        wd["m.down_proj.weight"])
    assert torch.allclose(residual.double().cpu(), h1, **tol(dtype, float(h1.abs().max())))
    assert torch.allclose(delta.double().cpu(), expected_delta, **tol(dtype, float(expected_delta.abs().max())))


# --------------------------------------------------------------------------- a toy architecture


@dataclass(frozen=True)
class ToyConfig:
    hidden_size: int
    vocab_size: int
    heads: int
    kv_heads: int
    head_dim: int
    inter_a: int
    inter_b: int
    decay: float
    eps: float
    theta: float

    @classmethod
    def from_dict(cls, data):
        return cls(**{k: data[k] for k in cls.__dataclass_fields__})


def register_toy():
    """Registers the toy mixer and the toy architecture with the package's public registries."""
    import miniserve_b200  # noqa: F401
    from miniserve_b200.config import register_architecture
    from miniserve_b200.parts import (LayerRun, LayerSpec, ModelSpec, ParamSpec, Part, PartSpec, StateNeed, register_mixer)

    @register_mixer("toy_decay")
    class ToyDecay(Part):
        """y_t = s_t with s_t = decay * s_(t-1) + W x_t: a running state of fixed size per request."""

        def __init__(self, *, prefix, hidden_size, decay):
            self.name, self.hidden, self.decay = prefix + "decay.weight", hidden_size, decay

        def param_specs(self):
            return [ParamSpec(self.name, (self.hidden, self.hidden))]

        def cache_need(self):
            return StateNeed((self.hidden,), torch.float32)

        def load(self, tensors):
            self.weight = tensors[self.name]

        def forward(self, x, ctx, cache):
            projected = (x.float() @ self.weight.float().T)
            if not ctx.host_state_slots:
                # inside a captured decode step nothing is known on the host: one token per row, slots on the device
                slots = ctx.state_slots.long()
                state = cache.states.index_select(0, slots) * self.decay + projected
                cache.states.index_copy_(0, slots, state)
                return state.to(x.dtype)
            out = torch.empty_like(projected)
            for r in range(ctx.n_requests):
                state = cache.states[ctx.host_state_slots[r]]
                for t in range(ctx.host_query_start[r], ctx.host_query_start[r + 1]):
                    state.mul_(self.decay).add_(projected[t])
                    out[t] = state
            return out.to(x.dtype)

    def build_spec(config: ToyConfig):
        rms = lambda name: PartSpec("rms", dict(name=name, size=config.hidden_size, eps=config.eps))
        attention = PartSpec("attention", dict(hidden_size=config.hidden_size, num_heads=config.heads, num_kv_heads=config.kv_heads,
                                               head_dim=config.head_dim, qk_norm=True, eps=config.eps,
                                               position=PartSpec("rope", dict(theta=config.theta))))
        layers = [
            LayerSpec("blocks.0.", attention, PartSpec("gated_mlp", dict(hidden_size=config.hidden_size, intermediate_size=config.inter_a)),
                      rms("norm_a.weight"), rms("norm_b.weight")),
            LayerSpec("blocks.1.", PartSpec("toy_decay", dict(hidden_size=config.hidden_size, decay=config.decay)),
                      PartSpec("gated_mlp", dict(hidden_size=config.hidden_size, intermediate_size=config.inter_b)),
                      rms("norm_a.weight"), rms("norm_b.weight")),
        ]
        # layer 0, layer 1, layer 0 again (a cache of its own), layer 1 again (a state of its own),
        # and layer 0 a third time reading the keys and values that its first run wrote
        order = [LayerRun(0), LayerRun(1), LayerRun(0), LayerRun(1), LayerRun(0, cache_of=0)]
        return ModelSpec(vocab_size=config.vocab_size, hidden_size=config.hidden_size, embedding_name="embed.weight",
                         layers=layers, order=order, final_norm=rms("final_norm.weight"), output_name="head.weight",
                         max_positions=4096)

    register_architecture("ToyHybridForCausalLM", ToyConfig, build_spec)


TOY = dict(architectures=["ToyHybridForCausalLM"], hidden_size=48, vocab_size=97, heads=3, kv_heads=1, head_dim=32, inter_a=80,
           inter_b=56, decay=0.7, eps=1e-5, theta=2e4)


def toy_plain_logits(tokens, w, c):
    """The toy model on one whole sequence, written out with the plain parts."""
    n = len(tokens)
    positions = torch.arange(n)
    x = w["embed.weight"][torch.tensor(tokens)]

    def attention(h, prefix, shared=None):
        q = (h @ w[prefix + "q_proj.weight"].T).view(n, c["heads"], c["head_dim"])
        q = plain.plain_rmsnorm(q, w[prefix + "q_norm.weight"], c["eps"])
        cos, sin = plain.plain_rope_tables(positions, c["head_dim"], c["theta"], torch.float64)
        q = plain.plain_apply_rope(q, cos, sin)
        if shared is None:
            k = (h @ w[prefix + "k_proj.weight"].T).view(n, c["kv_heads"], c["head_dim"])
            v = (h @ w[prefix + "v_proj.weight"].T).view(n, c["kv_heads"], c["head_dim"])
            k = plain.plain_apply_rope(plain.plain_rmsnorm(k, w[prefix + "k_norm.weight"], c["eps"]), cos, sin)
        else:
            k, v = shared
        out = plain.plain_attention(q, k, v, positions).reshape(n, -1) @ w[prefix + "o_proj.weight"].T
        return out, (k, v)

    def decay(h, prefix):
        projected = h @ w[prefix + "decay.weight"].T
        state, out = torch.zeros(c["hidden_size"], dtype=torch.float64), []
        for t in range(n):
            state = c["decay"] * state + projected[t]
            out.append(state)
        return torch.stack(out)

    def mlp(h, prefix):
        return plain.plain_swiglu(h, w[prefix + "gate_proj.weight"], w[prefix + "up_proj.weight"], w[prefix + "down_proj.weight"])

    first_cache = None
    for run, (layer, shared) in enumerate([(0, False), (1, False), (0, False), (1, False), (0, True)]):
        prefix = f"blocks.{layer}."
        normed = plain.plain_rmsnorm(x, w[prefix + "norm_a.weight"], c["eps"])
        if layer == 0:
            mixed, cache = attention(normed, prefix, first_cache if shared else None)
            if run == 0:
                first_cache = cache
        else:
            mixed = decay(normed, prefix)
        x = x + mixed
        x = x + mlp(plain.plain_rmsnorm(x, w[prefix + "norm_b.weight"], c["eps"]), prefix)
    return plain.plain_rmsnorm(x, w["final_norm.weight"], c["eps"]) @ w["head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_toy_architecture_with_stateful_mixer(tmp_path, dtype, cutting):
    from test_replay_gpu import CUTTINGS, build, replay

    register_toy()
    from miniserve_b200.weights import write_random_model

    folder = write_random_model(tmp_path / "toy", TOY, seed=9, matrix_std=0.08)
    runtime = None
    requests = {f"t{i}": helpers.random_tokens(TOY["vocab_size"], n, seed=600 + i) for i, n in enumerate((1, 9, 26, 40, 70))}
    steps = CUTTINGS[cutting](requests)
    pages = (helpers.max_live_tokens(steps, granule=16) + 7) // 8
    runtime = build(folder, dtype, pages, 8)
    groups = runtime.model.cache_groups
    assert [type(g.need).__name__ for g in groups] == ["PagedKVNeed", "StateNeed"] and [g.n_slots for g in groups] == [2, 2]
    assert [rc.writable for rc in runtime.model.run_caches] == [True, True, True, True, False]
    assert runtime.manager.prefix is None                      # per-request state rules out page sharing
    got = helpers.collect(steps, replay(runtime, steps))
    _, weights = plain.load_folder(folder, torch.float64)
    for rid, tokens in requests.items():
        expected = toy_plain_logits(tokens, weights, TOY)
        bound = (3e-5 if dtype == "float32" else 4e-2) * max(1.0, float(expected.abs().max()))
        for position, row in got[rid].items():
            assert float((row - expected[position]).abs().max()) <= bound, (rid, position)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_stateful_mixer_in_a_padded_decode_graph(tmp_path, dtype):
    """Three requests decode as the captured graph for four rows: the padding row runs the stateful mixer too,
    and must read and write the scratch state slot, not the slot of a live request."""
    from test_replay_gpu import build, replay

    register_toy()
    from miniserve_b200.weights import write_random_model

    folder = write_random_model(tmp_path / "toy", TOY, seed=9, matrix_std=0.08)
    prompt_lens = {"t0": 5, "t1": 1, "t2": 12}
    requests = {rid: helpers.random_tokens(TOY["vocab_size"], n + 9, seed=700 + i) for i, (rid, n) in enumerate(prompt_lens.items())}
    steps = helpers.cut_many_live(requests, prompt_lens, seed=1)
    runtime = build(folder, dtype, 12, 8, max_seqs=3, execution="cuda_graph", max_model_len=64)
    got = helpers.collect(steps, replay(runtime, steps))
    assert runtime.step_function.graph_replays > 0 and set(runtime.step_function.graphs) <= {1, 2, 4}
    assert 4 in runtime.step_function.graphs
    _, weights = plain.load_folder(folder, torch.float64)
    for rid, tokens in requests.items():
        expected = toy_plain_logits(tokens, weights, TOY)
        bound = (3e-5 if dtype == "float32" else 4e-2) * max(1.0, float(expected.abs().max()))
        assert sorted(got[rid]) == list(range(prompt_lens[rid] - 1, len(tokens)))
        for position, row in got[rid].items():
            assert float((row - expected[position]).abs().max()) <= bound, (rid, position)
    # the scratch slot took the padding rows' writes; no request was ever given it
    assert runtime.storage.scratch_slot == 3 and float(runtime.storage.states[1][:, 3].abs().max()) > 0


# --------------------------------------------------------------------------- a second toy: routing and another position encoding


@dataclass(frozen=True)
class RoutedConfig:
    hidden_size: int
    vocab_size: int
    heads: int
    kv_heads: int
    head_dim: int
    experts: int
    expert_size: int
    inter: int
    window: int
    amplitude: float
    eps: float
    theta: float

    @classmethod
    def from_dict(cls, data):
        return cls(**{k: data[k] for k in cls.__dataclass_fields__})


def sinusoid(positions, head_dim, amplitude, dtype):
    """amplitude * sin(position / 50^(j / d)) for j < d / 2, cos of the same for the other half."""
    half = head_dim // 2
    rates = 1.0 / (50.0 ** (torch.arange(half, dtype=torch.float64, device=positions.device) / half))
    angles = positions.to(torch.float64)[:, None] * rates[None, :]
    return (amplitude * torch.cat([angles.sin(), angles.cos()], dim=1)).to(dtype)


def register_routed_toy():
    """A feed-forward that routes every token to two of its experts and a position encoding that is added
    to queries and keys, registered with the package's public registries; and an architecture that uses
    them in one layer beside the package's own parts (a windowed attention with rotation, a gated MLP) in
    the other."""
    import miniserve_b200  # noqa: F401
    from miniserve_b200 import kernels
    from miniserve_b200.config import register_architecture
    from miniserve_b200.parts import (LayerRun, LayerSpec, ModelSpec, ParamSpec, Part, PartSpec,
                                      register_feed_forward, register_position)

    @register_position("toy_sinusoid")
    class AddedSinusoid(Part):
        """No fused form: the mixer norms the heads, calls ``apply`` and appends what comes back."""

        def __init__(self, *, head_dim, amplitude):
            self.head_dim, self.amplitude = head_dim, amplitude

        def fused_args(self, ctx):
            return None

        def apply(self, q, k, ctx):
            table = sinusoid(ctx.positions, self.head_dim, self.amplitude, torch.float32)[:, None, :]
            return (q.float() + table).to(q.dtype), (k.float() + table).to(k.dtype)

    @register_feed_forward("toy_routed")
    class RoutedExperts(Part):
        """y = sum over the two best experts e of p_e * down_e(relu(up_e x)), p = softmax of the two router
        scores; router scores in float32.  Every expert runs on every row and the unchosen ones are
        weighted 0, so nothing depends on the host knowing the choice."""

        def __init__(self, *, prefix, hidden_size, experts, expert_size):
            self.prefix, self.hidden, self.experts, self.size = prefix, hidden_size, experts, expert_size

        def param_specs(self):
            specs = [ParamSpec(self.prefix + "router.weight", (self.experts, self.hidden), "vector")]
            for e in range(self.experts):
                specs += [ParamSpec(f"{self.prefix}experts.{e}.up.weight", (self.size, self.hidden)),
                          ParamSpec(f"{self.prefix}experts.{e}.down.weight", (self.hidden, self.size))]
            return specs

        def load(self, tensors):
            self.router = tensors[self.prefix + "router.weight"].float()
            self.up = [tensors[f"{self.prefix}experts.{e}.up.weight"] for e in range(self.experts)]
            self.down = [tensors[f"{self.prefix}experts.{e}.down.weight"] for e in range(self.experts)]

        def forward(self, x, ctx):
            n = x.shape[0]
            scores = x.float() @ self.router.T
            best = scores.topk(2, dim=1)
            weights = torch.zeros_like(scores).scatter_(1, best.indices, best.values.softmax(dim=1))
            total = torch.zeros((n, self.hidden), dtype=torch.float32, device=x.device)
            hidden = torch.empty((n, self.size), dtype=x.dtype, device=x.device)
            out = torch.empty((n, self.hidden), dtype=x.dtype, device=x.device)
            for e in range(self.experts):
                kernels.linear(x, self.up[e], hidden)          # the package's own matrix product
                kernels.linear(hidden.clamp_(min=0), self.down[e], out)
                total += weights[:, e:e + 1] * out.float()
            return total.to(x.dtype)

    def build_spec(config: RoutedConfig):
        rms = lambda name: PartSpec("rms", dict(name=name, size=config.hidden_size, eps=config.eps))
        common = dict(hidden_size=config.hidden_size, num_heads=config.heads, num_kv_heads=config.kv_heads,
                      head_dim=config.head_dim, eps=config.eps)
        layers = [
            LayerSpec("blocks.0.",
                      PartSpec("attention", dict(common, qk_norm=True,
                                                 position=PartSpec("toy_sinusoid", dict(amplitude=config.amplitude)))),
                      PartSpec("toy_routed", dict(hidden_size=config.hidden_size, experts=config.experts,
                                                  expert_size=config.expert_size)),
                      rms("norm_a.weight"), rms("norm_b.weight")),
            LayerSpec("blocks.1.",
                      PartSpec("attention", dict(common, qk_norm=False, window=config.window,
                                                 position=PartSpec("rope", dict(theta=config.theta)))),
                      PartSpec("gated_mlp", dict(hidden_size=config.hidden_size, intermediate_size=config.inter)),
                      rms("norm_a.weight"), rms("norm_b.weight")),
        ]
        return ModelSpec(vocab_size=config.vocab_size, hidden_size=config.hidden_size, embedding_name="embed.weight",
                         layers=layers, order=[LayerRun(0), LayerRun(1)], final_norm=rms("final_norm.weight"),
                         output_name="head.weight", max_positions=4096)

    register_architecture("ToyRoutedForCausalLM", RoutedConfig, build_spec)


ROUTED = dict(architectures=["ToyRoutedForCausalLM"], hidden_size=80, vocab_size=131, heads=4, kv_heads=2, head_dim=16,
              experts=4, expert_size=40, inter=72, window=11, amplitude=0.6, eps=1e-6, theta=3e3)


def routed_plain_logits(tokens, w, c):
    """The routed toy on one whole sequence; also the smallest gap between the second and third router
    score over all tokens (how far the choice of experts is from a tie)."""
    n = len(tokens)
    positions = torch.arange(n)
    x = w["embed.weight"][torch.tensor(tokens)]
    heads, kv, d = c["heads"], c["kv_heads"], c["head_dim"]

    def project(h, prefix):
        return ((h @ w[prefix + "q_proj.weight"].T).view(n, heads, d), (h @ w[prefix + "k_proj.weight"].T).view(n, kv, d),
                (h @ w[prefix + "v_proj.weight"].T).view(n, kv, d))

    # layer 0: normed heads plus a sinusoid, all keys; two of four experts
    h = plain.plain_rmsnorm(x, w["blocks.0.norm_a.weight"], c["eps"])
    q, k, v = project(h, "blocks.0.")
    table = sinusoid(positions, d, c["amplitude"], torch.float64)[:, None, :]
    q = plain.plain_rmsnorm(q, w["blocks.0.q_norm.weight"], c["eps"]) + table
    k = plain.plain_rmsnorm(k, w["blocks.0.k_norm.weight"], c["eps"]) + table
    x = x + plain.plain_attention(q, k, v, positions).reshape(n, -1) @ w["blocks.0.o_proj.weight"].T
    h = plain.plain_rmsnorm(x, w["blocks.0.norm_b.weight"], c["eps"])
    scores = h @ w["blocks.0.router.weight"].T
    ranked = scores.sort(dim=1, descending=True)
    gap = float((ranked.values[:, 1] - ranked.values[:, 2]).min())
    weights = ranked.values[:, :2].softmax(dim=1)
    mixed = torch.zeros_like(x)
    for t in range(n):
        for j in range(2):
            e = int(ranked.indices[t, j])
            up, down = w[f"blocks.0.experts.{e}.up.weight"], w[f"blocks.0.experts.{e}.down.weight"]
            mixed[t] += weights[t, j] * (down @ (up @ h[t]).clamp(min=0))
    x = x + mixed
    # layer 1: rotation, a window of keys, gated MLP
    h = plain.plain_rmsnorm(x, w["blocks.1.norm_a.weight"], c["eps"])
    q, k, v = project(h, "blocks.1.")
    cos, sin = plain.plain_rope_tables(positions, d, c["theta"], torch.float64)
    q, k = plain.plain_apply_rope(q, cos, sin), plain.plain_apply_rope(k, cos, sin)
    x = x + plain.plain_attention(q, k, v, positions, window=c["window"]).reshape(n, -1) @ w["blocks.1.o_proj.weight"].T
    h = plain.plain_rmsnorm(x, w["blocks.1.norm_b.weight"], c["eps"])
    x = x + plain.plain_swiglu(h, w["blocks.1.gate_proj.weight"], w["blocks.1.up_proj.weight"], w["blocks.1.down_proj.weight"])
    return plain.plain_rmsnorm(x, w["final_norm.weight"], c["eps"]) @ w["head.weight"].T, gap


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_toy_architecture_with_routing_and_added_positions(tmp_path, dtype, cutting):
    """A feed-forward with routing and a position encoding without a fused form, both defined above, in
    one layer; the package's windowed attention (a cache group of its own, pages given back behind the
    window) and gated MLP in the other.  So that rounding cannot flip the choice of experts, the first
    columns of the embedding carry a clear mark of (token id mod experts) and the router reads it."""
    from safetensors.torch import load_file, save_file
    from test_replay_gpu import CUTTINGS, build, replay

    register_routed_toy()
    from miniserve_b200.weights import write_random_model

    folder = write_random_model(tmp_path / "routed", ROUTED, seed=12, matrix_std=0.08)
    tensors = {k: v.clone() for k, v in load_file(str(folder / "model.safetensors")).items()}
    experts = ROUTED["experts"]
    ids = torch.arange(ROUTED["vocab_size"])
    tensors["embed.weight"][:, :experts] = 0
    tensors["embed.weight"][ids, ids % experts] = 3.0
    second = (ids % experts + 1 + (ids // experts) % (experts - 1)) % experts      # another column, always
    tensors["embed.weight"][ids, second] = 1.5                                     # a clear second choice too
    router = tensors["blocks.0.router.weight"]
    router.copy_((router.float() - 1.0) * 0.5)                                     # (vectors are drawn around 1)
    router[:, :experts] += 2.0 * torch.eye(experts).to(router.dtype)
    save_file(tensors, str(folder / "model.safetensors"))

    requests = {f"t{i}": helpers.random_tokens(ROUTED["vocab_size"], n, seed=800 + i) for i, n in enumerate((2, 13, 31, 45, 66))}
    steps = CUTTINGS[cutting](requests)
    pages = (helpers.max_live_tokens(steps, granule=16) + 3) // 4
    runtime = build(folder, dtype, pages, 4)
    groups = runtime.model.cache_groups
    assert [(type(g.need).__name__, g.need.window) for g in groups] == [("PagedKVNeed", None), ("PagedKVNeed", ROUTED["window"])]
    got = helpers.collect(steps, replay(runtime, steps))
    _, weights = plain.load_folder(folder, torch.float64)
    for rid, tokens in requests.items():
        expected, gap = routed_plain_logits(tokens, weights, ROUTED)
        assert gap > 0.2, "the router's choice is too close to a tie for this test to mean anything"
        bound = (3e-5 if dtype == "float32" else 4e-2) * max(1.0, float(expected.abs().max()))
        for position, row in got[rid].items():
            assert float((row - expected[position]).abs().max()) <= bound, (rid, position)
    runtime.manager.check_invariants()


# --------------------------------------------------------------------------- a third toy: the frame around the layers, and scores with a bias


BIASED = dict(architectures=["ToyBiasedForCausalLM"], hidden_size=64, vocab_size=113, heads=4, kv_heads=2, head_dim=32,
              inter=96, eps=1e-6, embedding_scale=8.0, logit_scale=0.5, logit_softcap=6.0, score_softcap=4.0,
              slopes=[0.25, 0.125, 0.0625, 0.03125])


@dataclass(frozen=True)
class BiasedConfig:
    hidden_size: int
    vocab_size: int
    heads: int
    kv_heads: int
    head_dim: int
    inter: int
    eps: float
    embedding_scale: float
    logit_scale: float
    logit_softcap: float
    score_softcap: float
    slopes: tuple

    @classmethod
    def from_dict(cls, data):
        return cls(**{k: (tuple(data[k]) if k == "slopes" else data[k]) for k in cls.__dataclass_fields__})


def register_biased_toy():
    """An architecture made of the package's own parts only, with options that Qwen3 leaves at their defaults:
    embeddings scaled as they enter the stream, logits scaled and soft-capped, and an attention without any
    rotation whose scores are soft-capped and biased by the distance between query and key."""
    import miniserve_b200  # noqa: F401
    from miniserve_b200.config import register_architecture
    from miniserve_b200.parts import LayerRun, LayerSpec, ModelSpec, PartSpec

    def build_spec(config: BiasedConfig):
        rms = lambda name: PartSpec("rms", dict(name=name, size=config.hidden_size, eps=config.eps))
        attention = PartSpec("attention", dict(
            hidden_size=config.hidden_size, num_heads=config.heads, num_kv_heads=config.kv_heads, head_dim=config.head_dim,
            qk_norm=False, eps=config.eps, position=PartSpec("none"), score_softcap=config.score_softcap,
            score_bias_slopes=config.slopes))
        layers = [LayerSpec(f"blocks.{i}.", attention,
                            PartSpec("gated_mlp", dict(hidden_size=config.hidden_size, intermediate_size=config.inter)),
                            rms("norm_a.weight"), rms("norm_b.weight")) for i in range(2)]
        return ModelSpec(vocab_size=config.vocab_size, hidden_size=config.hidden_size, embedding_name="embed.weight",
                         layers=layers, order=[LayerRun(0), LayerRun(1)], final_norm=rms("final_norm.weight"),
                         output_name=None, max_positions=1024, embedding_scale=config.embedding_scale,
                         logit_scale=config.logit_scale, logit_softcap=config.logit_softcap)

    register_architecture("ToyBiasedForCausalLM", BiasedConfig, build_spec)


def biased_plain_logits(tokens, w, c):
    n = len(tokens)
    heads, kv, d = c["heads"], c["kv_heads"], c["head_dim"]
    positions = torch.arange(n, dtype=torch.float64)
    distance = positions[None, :] - positions[:, None]                       # key position - query position
    causal = distance <= 0
    x = c["embedding_scale"] * w["embed.weight"][torch.tensor(tokens)]
    for layer in range(2):
        prefix = f"blocks.{layer}."
        h = plain.plain_rmsnorm(x, w[prefix + "norm_a.weight"], c["eps"])
        q = (h @ w[prefix + "q_proj.weight"].T).view(n, heads, d)
        k = (h @ w[prefix + "k_proj.weight"].T).view(n, kv, d)
        v = (h @ w[prefix + "v_proj.weight"].T).view(n, kv, d)
        attended = torch.zeros(n, heads, d, dtype=torch.float64)
        for head in range(heads):
            scores = (q[:, head] @ k[:, head // (heads // kv)].T) * d ** -0.5
            scores = c["score_softcap"] * torch.tanh(scores / c["score_softcap"]) + c["slopes"][head] * distance
            scores = scores.masked_fill(~causal, float("-inf"))
            attended[:, head] = scores.softmax(dim=1) @ v[:, head // (heads // kv)]
        x = x + attended.reshape(n, -1) @ w[prefix + "o_proj.weight"].T
        h = plain.plain_rmsnorm(x, w[prefix + "norm_b.weight"], c["eps"])
        x = x + plain.plain_swiglu(h, w[prefix + "gate_proj.weight"], w[prefix + "up_proj.weight"], w[prefix + "down_proj.weight"])
    logits = c["logit_scale"] * (plain.plain_rmsnorm(x, w["final_norm.weight"], c["eps"]) @ w["embed.weight"].T)
    return c["logit_softcap"] * torch.tanh(logits / c["logit_softcap"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cutting", ["whole", "tail", "mixed"])
def test_toy_architecture_with_scaled_frame_and_biased_scores(tmp_path, dtype, cutting):
    """Scaled embeddings, scaled and soft-capped logits (fields of the model's spec), and an attention whose
    position encoding acts on the scores (a soft cap and a per-head bias by distance, options of the attention
    part): an architecture registered from here, replayed in three cuttings against plain code above."""
    from test_replay_gpu import CUTTINGS, build, replay

    register_biased_toy()
    from miniserve_b200.weights import write_random_model

    folder = write_random_model(tmp_path / "biased", BIASED, seed=21, matrix_std=0.08)
    requests = {f"t{i}": helpers.random_tokens(BIASED["vocab_size"], n, seed=900 + i) for i, n in enumerate((1, 17, 40, 75))}
    steps = CUTTINGS[cutting](requests)
    pages = (helpers.max_live_tokens(steps, granule=16) + 7) // 8
    runtime = build(folder, dtype, pages, 8)
    assert runtime.attention_kernels[0]["decode"] == "general"           # modified scores: the general kernel, said at build
    got = helpers.collect(steps, replay(runtime, steps))
    _, weights = plain.load_folder(folder, torch.float64)
    for rid, tokens in requests.items():
        expected = biased_plain_logits(tokens, weights, BIASED)
        assert float(expected.abs().max()) > 1.0                          # the soft cap of the logits is in play
        bound = (3e-5 if dtype == "float32" else 4e-2) * max(1.0, float(expected.abs().max()))
        for position, row in got[rid].items():
            assert float((row - expected[position]).abs().max()) <= bound, (rid, position)
