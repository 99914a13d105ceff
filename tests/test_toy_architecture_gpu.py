"""An architecture defined here, in the test: registered, built, loaded and stepped with no change
to the framework's files.  It is a toy, not anyone's model.  Its layers differ in kind:

  0  a mixer with a state of its own (a decaying running sum kept in a per-request slot) that walks a step's
     tokens in chunks of 24, cut by a step planner of its own: the step function packs and uploads what the
     planner returns without knowing what a chunk is
  1  full attention with q/k norms and full rotation
  2  attention with a window of 20 positions and a position encoding of the test's own: half of each head is
     rotated, by angles of positions squeezed by a factor plus a phase per frequency; its feed-forward is
     routed: a float32 router picks two of three small experts per token
  3  attention without k/v projections that reads the pages layer 1 wrote

and its order names layer 0 twice: [0, 1, 2, 3, 0].  Each call of layer 0 keeps its own state.
"""
import json
from dataclasses import asdict, dataclass

import pytest
import torch

from tests import harness
from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu


@dataclass(frozen=True)
class ToyConfig:
    vocab_size: int = 211
    width: int = 48
    state_width: int = 24
    decay: float = 0.9
    heads: int = 4
    kv_heads: int = 2
    head_dim: int = 16
    window: int = 20
    partial_rotary: int = 8
    squeeze: float = 2.5
    theta: float = 10000.0
    eps: float = 1e-5
    inner: int = 72
    experts: int = 3
    experts_per_token: int = 2
    expert_inner: int = 40
    max_positions: int = 512

    architecture = "ToyStateLM"
    model_type = "toy_state"

    @classmethod
    def from_dict(cls, data):
        return cls(**{k: v for k, v in data.items() if k in cls.__dataclass_fields__})

    def to_dict(self):
        return asdict(self) | {"architectures": [self.architecture], "model_type": self.model_type}


def squeezed_angles(positions, rotary_dim, theta, squeeze):
    """angle[p, j] = p / squeeze / theta^(2j / rotary_dim) + 0.1 j: the toy's own position encoding."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))
    return positions.float()[:, None] / squeeze * inv_freq[None, :] + 0.1 * torch.arange(rotary_dim // 2).float()


SCAN_CHUNK = 24


def make_parts():
    import numpy as np
    from qwen_inference_lab_b200.parts import FeedForward, Mixer, Param, PositionEncoding, StateSpec, StepPlanner

    class ScanPlanner(StepPlanner):
        """Segments cut into chunks of at most SCAN_CHUNK tokens: (first token, tokens, state slot) each."""
        key = "toy_scan"

        def plan(self, segments):
            chunks = [(int(first) + off, min(SCAN_CHUNK, int(n) - off), int(row))
                      for first, n, row in zip(segments.first, segments.lens, segments.rows)
                      for off in range(0, int(n), SCAN_CHUNK)]
            return dict(chunks=np.array(chunks, dtype=np.int64).reshape(-1))

    scan_planner = ScanPlanner()

    class SqueezedRotation(PositionEncoding):
        """Another position encoding is another table of cosines and sines."""
        graph_safe = True

        def __init__(self, rotary_dim, theta, squeeze, max_positions):
            self.rotary_dim, self.theta, self.squeeze, self.max_positions = rotary_dim, theta, squeeze, max_positions

        def finalize(self, device, dtype):
            angles = squeezed_angles(torch.arange(self.max_positions), self.rotary_dim, self.theta, self.squeeze)
            self.table = torch.cat((angles.cos(), angles.sin()), dim=-1).to(dtype).float().contiguous().to(device)

    class RoutedFeedForward(FeedForward):
        """Router logits in float32, softmax over the chosen experts, tokens gathered per expert and
        put back in their order before the residual is added."""

        def __init__(self, width, inner, experts, per_token, *, name):
            self.per_token, self.name = per_token, name
            self.router = Param((experts, width), std=0.5, keep_32bit=True)
            self.gate = [Param((inner, width), std=0.1) for _ in range(experts)]
            self.up = [Param((inner, width), std=0.1) for _ in range(experts)]
            self.down = [Param((width, inner), std=0.1) for _ in range(experts)]

        def named_params(self):
            names = {self.name + ".router": self.router}
            for e, (g, u, d) in enumerate(zip(self.gate, self.up, self.down)):
                names.update({f"{self.name}.experts.{e}.gate": g, f"{self.name}.experts.{e}.up": u,
                              f"{self.name}.experts.{e}.down": d})
            return names

        def forward(self, ctx, x, residual=None):
            logits = x.float() @ self.router.data.float().t()
            top, chosen = logits.topk(self.per_token, dim=-1)
            weights = torch.softmax(top, dim=-1)
            out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            for e in range(len(self.gate)):
                token, slot = (chosen == e).nonzero(as_tuple=True)
                if token.numel() == 0:
                    continue
                xe = x[token].float()
                hidden = torch.nn.functional.silu(xe @ self.gate[e].data.float().t()) * (xe @ self.up[e].data.float().t())
                out.index_add_(0, token, (hidden @ self.down[e].data.float().t()) * weights[token, slot].unsqueeze(1))
            return (out if residual is None else residual.float() + out).to(x.dtype)

    class RunningStateMixer(Mixer):
        """h_t = decay * h_{t-1} + W_in x_t ;  y_t = W_out h_t.  The state h lives in the request's slot."""

        def __init__(self, width, state_width, decay, *, name):
            self.decay, self.state_width = decay, state_width
            self.w_in, self.w_out = Param((state_width, width), std=0.2), Param((width, state_width), std=0.2)
            self.name = name

        def named_params(self):
            return {self.name + ".w_in": self.w_in, self.name + ".w_out": self.w_out}

        def cache_spec(self):
            return StateSpec((self.state_width,), torch.float32)

        def step_planners(self):
            return {**super().step_planners(), scan_planner.key: scan_planner}

        def forward(self, ctx, x, cache, residual=None):
            u = x.float() @ self.w_in.data.float().t()
            h_all = torch.empty_like(u)
            plan = ctx.plans["toy_scan"]
            assert plan.count["chunks"] == plan.array["chunks"].numel() and plan.array["chunks"].dtype == torch.int32
            chunks = plan.array["chunks"].view(-1, 3).tolist()      # from the device: what the step function uploaded
            assert all(0 < length <= SCAN_CHUNK for _, length, _ in chunks)
            assert sum(length for _, length, _ in chunks) == ctx.n_tokens
            for start, length, row in chunks:
                h = cache.slots[row]                                 # a later chunk of a segment goes on from the slot
                for t in range(start, start + length):
                    h = self.decay * h + u[t]
                    h_all[t] = h
                cache.slots[row] = h
            y = (h_all @ self.w_out.data.float().t()).to(x.dtype)
            return y if residual is None else (residual.float() + y.float()).to(x.dtype)

    return RunningStateMixer, RoutedFeedForward, SqueezedRotation


def build_toy(config):
    from qwen_inference_lab_b200.parts import (DecoderModel, GatedMLP, GroupedQueryAttention, LayerCall, Linear,
                                               PreNormBlock, RMSNorm, RotaryEmbedding, TokenEmbedding)
    RunningStateMixer, RoutedFeedForward, SqueezedRotation = make_parts()
    w, d = config.width, config.head_dim
    def block(i, mixer, routed=False):
        feed_forward = RoutedFeedForward(w, config.expert_inner, config.experts, config.experts_per_token,
                                         name=f"blocks.{i}.ff") if routed else \
            GatedMLP(w, config.inner, names={k: f"blocks.{i}.ff.{k}" for k in ("gate", "up", "down")})
        return PreNormBlock(RMSNorm(w, config.eps, name=f"blocks.{i}.norm_a"), mixer,
                            RMSNorm(w, config.eps, name=f"blocks.{i}.norm_b"), feed_forward)
    def attention(i, **kw):
        names = {k: f"blocks.{i}.attn.{k}" for k in ("q", "k", "v", "o", "q_norm", "k_norm")}
        return GroupedQueryAttention(w, config.heads, config.kv_heads, d, names=names, **kw)
    layers = [
        block(0, RunningStateMixer(w, config.state_width, config.decay, name="blocks.0.state")),
        block(1, attention(1, qk_norm_eps=config.eps, position=RotaryEmbedding(d, config.theta, config.max_positions))),
        block(2, attention(2, qk_norm_eps=config.eps, window=config.window, bias=True,
                           position=SqueezedRotation(config.partial_rotary, config.theta, config.squeeze,
                                                     config.max_positions)),
              routed=True),
        block(3, attention(3, reads_shared_cache=True, position=RotaryEmbedding(d, config.theta, config.max_positions))),
    ]
    embedding = TokenEmbedding(config.vocab_size, w, name="embed")
    return DecoderModel(config=config, embedding=embedding, layers=layers,
                        order=[LayerCall(0), LayerCall(1), LayerCall(2), LayerCall(3, reads_cache_of=1), LayerCall(0)],
                        final_norm=RMSNorm(w, config.eps, name="final_norm"),
                        head=Linear(w, config.vocab_size, name="head", weight=embedding.weight),
                        max_positions=config.max_positions)


# ------------------------------------------------------------------ the toy, written plainly for whole sequences
def toy_plain_logits(tokens, w, c: ToyConfig, dtype=torch.float32):
    """``dtype``: the activation dtype; the state mixer and the routed feed-forward compute in float32 and round
    their sum with the residual once, as the toy's parts above do."""
    T = len(tokens)
    x = w["embed.weight"].to(dtype)[torch.as_tensor(tokens)]
    positions = torch.arange(T)
    kv_of_layer1 = {}

    def routed_ff(i, x):
        n = plain.rms_norm(x, w[f"blocks.{i}.norm_b.weight"], c.eps).float()
        logits = n @ w[f"blocks.{i}.ff.router"].t()
        out = torch.zeros(x.shape)
        for t in range(T):                      # one token at a time: the plainest form
            top, chosen = logits[t].topk(c.experts_per_token)
            share = torch.softmax(top, dim=-1)
            for e, p in zip(chosen.tolist(), share):
                pre = f"blocks.{i}.ff.experts.{e}."
                hidden = torch.nn.functional.silu(n[t] @ w[pre + "gate"].t()) * (n[t] @ w[pre + "up"].t())
                out[t] += p * (hidden @ w[pre + "down"].t())
        return (x.float() + out).to(x.dtype)

    def ff(i, x):
        if i == 2:
            return routed_ff(i, x)
        n = plain.rms_norm(x, w[f"blocks.{i}.norm_b.weight"], c.eps)
        gate = torch.nn.functional.silu(plain.linear(n, w[f"blocks.{i}.ff.gate.weight"]))
        return x + plain.linear(gate * plain.linear(n, w[f"blocks.{i}.ff.up.weight"]), w[f"blocks.{i}.ff.down.weight"])

    def state_layer(x):
        n = plain.rms_norm(x, w["blocks.0.norm_a.weight"], c.eps).float()
        u = n @ w["blocks.0.state.w_in"].t()
        h, rows = torch.zeros(c.state_width), []
        for t in range(T):
            h = c.decay * h + u[t]
            rows.append(h)
        mixed = (torch.stack(rows) @ w["blocks.0.state.w_out"].t()).to(x.dtype)
        return ff(0, (x.float() + mixed.float()).to(x.dtype))

    def rotate_part(v, rotary_dim):
        angles = plain.rotary_angles(positions, rotary_dim, c.theta) if rotary_dim == c.head_dim else \
            squeezed_angles(positions, rotary_dim, c.theta, c.squeeze)
        return torch.cat((plain.rotate(v[..., :rotary_dim], angles), v[..., rotary_dim:]), dim=-1)

    def attention_layer(i, x, norms, rotary_dim, window=0, shared=False, bias=False):
        n = plain.rms_norm(x, w[f"blocks.{i}.norm_a.weight"], c.eps)
        b = lambda k: w.get(f"blocks.{i}.attn.{k}.bias") if bias else None
        q = plain.linear(n, w[f"blocks.{i}.attn.q.weight"], b("q")).reshape(T, c.heads, c.head_dim)
        if norms:
            q = plain.rms_norm(q, w[f"blocks.{i}.attn.q_norm.weight"], c.eps)
        q = rotate_part(q, rotary_dim)
        if shared:
            k, v = kv_of_layer1["k"], kv_of_layer1["v"]
        else:
            k = plain.linear(n, w[f"blocks.{i}.attn.k.weight"], b("k")).reshape(T, c.kv_heads, c.head_dim)
            v = plain.linear(n, w[f"blocks.{i}.attn.v.weight"], b("v")).reshape(T, c.kv_heads, c.head_dim)
            if norms:
                k = plain.rms_norm(k, w[f"blocks.{i}.attn.k_norm.weight"], c.eps)
            k = rotate_part(k, rotary_dim)
            if i == 1:
                kv_of_layer1.update(k=k, v=v)
        out = plain.causal_attention(q, k, v, c.head_dim ** -0.5, window=window).reshape(T, -1)
        return ff(i, x + plain.linear(out, w[f"blocks.{i}.attn.o.weight"], b("o")))

    x = state_layer(x)
    x = attention_layer(1, x, norms=True, rotary_dim=c.head_dim)
    x = attention_layer(2, x, norms=True, rotary_dim=c.partial_rotary, window=c.window, bias=True)
    x = attention_layer(3, x, norms=False, rotary_dim=c.head_dim, shared=True)
    x = state_layer(x)
    return plain.linear(plain.rms_norm(x, w["final_norm.weight"], c.eps), w["embed.weight"]).float()


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    from qwen_inference_lab_b200.config import registry
    from qwen_inference_lab_b200.weights import SafetensorsFile, write_model_folder
    registry.register(ToyConfig.architecture, ToyConfig.model_type, ToyConfig, build_toy)
    try:
        config = ToyConfig()
        folder = write_model_folder(config, 11, tmp_path_factory.mktemp("toy"))
        with SafetensorsFile(folder / "model.safetensors") as f:
            weights = {name: f.tensor(name).float().clone() for name in f.keys()}
        yield config, folder, weights
    finally:
        registry.unregister(ToyConfig.architecture)


def engine_parts(folder, dtype, num_pages=40, page_size=4):
    from qwen_inference_lab_b200.cache import CacheManager
    from qwen_inference_lab_b200.engine import StepRunner
    from qwen_inference_lab_b200.loading import load_model
    model = load_model(folder, device="cuda", dtype=dtype)
    cache = CacheManager(model.cache_specs(), num_pages=num_pages, page_size=page_size, max_requests=4,
                         max_context=model.max_positions, dtype=dtype, device=model.device, max_step_tokens=64)
    cache.poison()
    return model, cache, StepRunner(model, cache)


def test_toy_is_registered_built_and_loaded(toy):
    config, folder, weights = toy
    from qwen_inference_lab_b200.config import registry
    entry, read_back = registry.read_model_config(folder)
    assert entry.name == "ToyStateLM" and read_back == config
    model, cache, runner = engine_parts(folder, torch.float32)
    assert not model.is_graph_safe() and not runner.use_graphs          # the toy mixer works on the host
    assert len(cache.state_groups) == 1 and cache.state_groups[0][1] == [0, 4]      # layer 0 twice: two states
    assert [g.spec.window for g in cache.kv_groups] == [0, 20] and cache.specs[3] is None
    assert "blocks.3.attn.k.weight" not in weights and "blocks.0.state.w_in" in weights
    assert "blocks.2.ff.experts.2.down" in weights and "blocks.2.ff.gate.weight" not in weights


@pytest.mark.parametrize("schedule", ["whole", "tail_decode", "chunks", "mixed"])
def test_toy_steps_like_its_plain_form_under_every_cut(toy, schedule):
    config, folder, weights = toy
    requests = {f"r{i}": torch.randint(0, config.vocab_size, (n,), generator=torch.Generator().manual_seed(i)).tolist()
                for i, n in enumerate((150, 9, 64, 33, 90))}
    makers = dict(whole=harness.whole_schedule, tail_decode=harness.tail_decode_schedule,
                  chunks=harness.chunk_schedule, mixed=harness.mixed_schedule)
    # pages: the full-attention group must hold whole requests, up to four at a time in the mixed run
    model, cache, runner = engine_parts(folder, torch.float32, num_pages=4 * 38 if schedule == "mixed" else 38)
    actual = harness.run_schedule(runner, cache, makers[schedule](requests))
    assert all(len(g.free) == g.capacity for g in cache.kv_groups)
    expected = {(rid, p): row for rid, tokens in requests.items()
                for p, row in enumerate(toy_plain_logits(tokens, weights, config))}
    harness.assert_rows_close(actual, expected, torch.float32, f"toy {schedule}")


def test_window_group_holds_few_pages_while_a_long_request_runs(toy):
    config, folder, _ = toy
    model, cache, runner = engine_parts(folder, torch.float32, num_pages=60)
    tokens = torch.randint(0, config.vocab_size, (200,), generator=torch.Generator().manual_seed(9)).tolist()
    schedule = harness.chunk_schedule({"r": tokens}, sizes=(16, 7, 2, 5))
    from qwen_inference_lab_b200.engine import StepEntry
    cache.admit("r")
    for entries, _ in schedule:
        runner.run([StepEntry(rid, t, []) for rid, t, _ in entries])
        windowed = cache.kv_groups[1]
        assert sum(1 for p in windowed.tables["r"] if p >= 0) <= (config.window + 16) // 4 + 2
    assert sum(1 for p in cache.kv_groups[0].tables["r"] if p >= 0) == 50
    cache.release("r")
    cache.check_invariants()


def test_toy_in_bfloat16_under_two_cuts(toy):
    """bfloat16: whole and in portions, judged like the replay tests: against the plain float32 rows with the plain
    form's own bfloat16 arithmetic as the yardstick, and by the best token where it is clear."""
    config, folder, weights = toy
    requests = {"a": torch.randint(0, config.vocab_size, (70,), generator=torch.Generator().manual_seed(3)).tolist()}
    model, cache, runner = engine_parts(folder, torch.bfloat16)
    truth = {("a", p): row for p, row in enumerate(toy_plain_logits(requests["a"], weights, config))}
    yardstick = {("a", p): row for p, row in enumerate(toy_plain_logits(requests["a"], weights, config, torch.bfloat16))}
    for name, schedule in (("whole", harness.whole_schedule), ("chunks", harness.chunk_schedule)):
        rows = harness.run_schedule(runner, cache, schedule(requests))
        harness.assert_rows_close(rows, truth, torch.bfloat16, f"toy bfloat16 {name}", yardstick)
