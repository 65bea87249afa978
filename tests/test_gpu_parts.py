"""Each part of a layer alone against its plain twin, built directly from its spec with random
tensors, and three toy architectures registered from here, without touching the package: one with a toy
mixer (state of its own), a layer that runs twice and a run that reads another run's cache; one with a
feed-forward that routes tokens to experts and a position encoding that is added to the stream; one whose
layers take turns between attention over every key and over a window (two cache groups)."""
import dataclasses
import json
import os

import numpy as np
import pytest
import torch

from plain import llama_plain as P

pytestmark = pytest.mark.gpu


def runtime(dtype):
    from burn_lm_b200.parts import Runtime
    return Runtime(dtype, torch.device("cuda"))


def step_for(lengths, starts=None, slots=None):
    """A StepContext for sequences of the given new lengths."""
    from burn_lm_b200.engine import Workspace
    from burn_lm_b200.parts import StepContext
    starts = starts or [0] * len(lengths)
    slots = slots or list(range(len(lengths)))
    cu = [0]
    for n in lengths:
        cu.append(cu[-1] + n)
    dev = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")
    return StepContext(
        n_tokens=cu[-1], n_seqs=len(lengths), max_q_len=max(lengths), max_kv_len=max(s + n for s, n in zip(starts, lengths)),
        tokens=dev([0] * cu[-1]), token_seq=dev([s for s, n in enumerate(lengths) for _ in range(n)]),
        token_pos=dev([starts[s] + t for s, n in enumerate(lengths) for t in range(n)]), cu_seqlens=dev(cu),
        slot_of_seq=dev(slots), start_pos=dev(starts), want_rows=None, n_want=0, workspace=Workspace(torch.device("cuda")),
        host={"cu_seqlens": cu, "slots": slots, "start_pos": starts})


# largest error of an output row relative to the row's largest value (outputs may cross zero, so an
# element-wise relative tolerance would mean nothing)
TOL = {torch.float32: 1e-5, torch.bfloat16: 3e-2}   # bfloat16: the bound used for logits everywhere


def assert_rows_close(got, want, dtype):
    from tiny import row_error
    err = row_error(got.double().cpu().numpy(), want)
    assert err.max() < TOL[dtype], (float(err.max()), int(err.argmax()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rms_norm_part(dtype):
    from burn_lm_b200.parts import RMSNorm, RMSNormSpec
    part = RMSNorm(RMSNormSpec(size=88, eps=2e-6), {"weight": "g"}, runtime(dtype))
    assert [(s.name, s.shape) for s in part.tensor_specs()] == [("g", (88,))]
    g = (1 + 0.1 * torch.randn(88)).to(dtype).cuda()
    part.bind({"g": g})
    resid = torch.randn(9, 88, device="cuda")
    delta = torch.randn(9, 88, device="cuda").to(dtype)
    want = P.rms_norm((resid.double() + delta.double()).cpu().numpy(), g.double().cpu().numpy(), 2e-6)
    got = part.add_norm(resid, delta)
    assert_rows_close(got, want, dtype)


def test_rotary_part_frequencies():
    from burn_lm_b200.parts import Llama3Scaling, Rotary, RotarySpec
    spec = RotarySpec(head_dim=48, theta=77777.0, scaling=Llama3Scaling(5.0, 1.0, 3.0, 100))
    part = Rotary(spec, {}, runtime(torch.float32))
    want = P.llama3_frequency_scaling(P.rope_inverse_frequencies(48, 77777.0), 5.0, 1.0, 3.0, 100)
    inv, rot, inter = part.rotation()
    assert rot == 48 and not inter
    np.testing.assert_allclose(inv.cpu().numpy(), want, rtol=1e-14)
    part2 = Rotary(RotarySpec(head_dim=48, theta=10.0, rotary_dim=16, interleaved=True), {}, runtime(torch.float32))
    assert part2.rotation()[1:] == (16, True) and part2.rotation()[0].numel() == 8


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("interleaved", [False, True])
def test_attention_part(dtype, interleaved):
    """The mixer alone with a cache of its own: two prompts, then both continue by single tokens."""
    from burn_lm_b200.cache import Cache
    from burn_lm_b200.parts import Attention, AttentionSpec, RotarySpec
    from burn_lm_b200.plan import PartPlan, ScheduleEntry
    D, H, KV, hd = 72, 6, 3, 16
    spec = AttentionSpec(D, H, KV, hd, PartPlan("rotary", RotarySpec(head_dim=hd, theta=500.0, interleaved=interleaved)))
    part = Attention(spec, {"q": "q", "k": "k", "v": "v", "o": "o"}, runtime(dtype))
    g = torch.Generator().manual_seed(1)
    w = {n: (0.3 * torch.randn(*s, generator=g)).to(dtype).cuda()
         for n, s in (("q", (H * hd, D)), ("k", (KV * hd, D)), ("v", (KV * hd, D)), ("o", (D, H * hd)))}
    part.bind(w)
    cache = Cache([part.cache_need()], [ScheduleEntry(0)], 64 * 4, 2, 128, dtype, torch.device("cuda"))
    lens = [70, 9]
    xs = [(torch.randn(n + 5, D, generator=g)).to(dtype).cuda() for n in lens]
    slots = [cache.acquire(), cache.acquire()]
    wn = {n: t.double().cpu().numpy() for n, t in w.items()}
    inv = P.rope_inverse_frequencies(hd, 500.0)
    want = [P.attention(x.double().cpu().numpy(), wn["q"], wn["k"], wn["v"], wn["o"], H, KV, hd, inv,
                        "interleaved" if interleaved else "half") for x in xs]
    cache.reserve([(s, n) for s, n in zip(slots, lens)])
    out = part.forward(torch.cat([x[:n] for x, n in zip(xs, lens)]), step_for(lens, slots=slots), cache.view(0))
    got = [out[:70], out[70:]]
    for s, n in zip(slots, lens):
        cache.set_length(s, n)
    for t in range(5):
        starts = [n + t for n in lens]
        cache.reserve([(s, st + 1) for s, st in zip(slots, starts)])
        o = part.forward(torch.stack([x[st] for x, st in zip(xs, starts)]), step_for([1, 1], starts, slots), cache.view(0))
        got = [torch.cat([gg, o[i:i + 1]]) for i, gg in enumerate(got)]
    for gg, ww in zip(got, want):
        assert_rows_close(gg, ww, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part(dtype):
    from burn_lm_b200.parts import SwiGLU, SwiGLUSpec
    part = SwiGLU(SwiGLUSpec(hidden_size=40, intermediate_size=104), {"gate": "g", "up": "u", "down": "d"}, runtime(dtype))
    gen = torch.Generator().manual_seed(2)
    w = {"g": torch.randn(104, 40, generator=gen) * 0.3, "u": torch.randn(104, 40, generator=gen) * 0.3,
         "d": torch.randn(40, 104, generator=gen) * 0.3}
    w = {k: v.to(dtype).cuda() for k, v in w.items()}
    part.bind(w)
    x = torch.randn(7, 40, generator=gen).to(dtype).cuda()
    want = P.feed_forward(x.double().cpu().numpy(), *(w[k].double().cpu().numpy() for k in ("g", "u", "d")))
    assert_rows_close(part.forward(x, None), want, dtype)


def test_a_layer_stored_in_32_bit_inside_a_bfloat16_model():
    """A tensor stored in 32-bit stays so: its products run through the fp32 kernel."""
    from burn_lm_b200.parts import SwiGLU, SwiGLUSpec
    part = SwiGLU(SwiGLUSpec(hidden_size=40, intermediate_size=104), {"gate": "g", "up": "u", "down": "d"},
                  runtime(torch.bfloat16))
    gen = torch.Generator().manual_seed(3)
    w = {"g": torch.randn(104, 40, generator=gen).cuda(), "u": torch.randn(104, 40, generator=gen).cuda(),
         "d": torch.randn(40, 104, generator=gen).cuda()}
    part.bind(w)
    assert part.gate_up.weight.dtype == torch.float32
    x = torch.randn(7, 40, generator=gen).to(torch.bfloat16).cuda()
    want = P.feed_forward(x.double().cpu().numpy(), *(w[k].double().cpu().numpy() for k in ("g", "u", "d")))
    got = part.forward(x, None)
    assert got.dtype == torch.bfloat16
    assert_rows_close(got, want, torch.bfloat16)


# --------------------------------------------------------------------------------------------------
# a toy architecture, registered from the test
# --------------------------------------------------------------------------------------------------
@dataclasses.dataclass(frozen=True)
class DecaySpec:
    hidden_size: int
    decay: float


def register_toy():
    """A mixer with fixed-size state of its own: s_t = decay * s_{t-1} + x_t W_in; out_t = s_t W_out.
    Written with torch operations here in the test; it uses the cache's state block of its slot."""
    from burn_lm_b200 import register_architecture, register_part, Architecture, TensorSpec
    from burn_lm_b200.config import KeyReader
    from burn_lm_b200.parts import CacheNeed, Part, RMSNormSpec, SwiGLUSpec, AttentionSpec, NoPositionSpec, EmbeddingSpec, HeadSpec
    from burn_lm_b200.plan import ModelPlan, PartPlan, ScheduleEntry, prenorm_layer
    from burn_lm_b200 import registry

    if "ToyDecayLM" in [a.name for a in registry.architectures()]:
        return

    @register_part("mixer", "toy_decay")
    class DecayMixer(Part):
        family = "mixer"

        def tensor_specs(self):
            d = self.spec.hidden_size
            return [TensorSpec(self.tensor_names["w_in"], (d, d), init="normal:0.1"),
                    TensorSpec(self.tensor_names["w_out"], (d, d), init="normal:0.1")]

        def bind(self, loaded):
            self.w_in = loaded[self.tensor_names["w_in"]].float()
            self.w_out = loaded[self.tensor_names["w_out"]].float()

        def cache_need(self):
            return CacheNeed("state", state_shape=(self.spec.hidden_size,), state_dtype="float32")

        def forward(self, x, step, cache):
            u = x.float() @ self.w_in.T
            out = torch.empty_like(u)
            cu, slots = step.host["cu_seqlens"], step.host["slots"]
            for s, slot in enumerate(slots):
                state = cache.state[slot]
                for t in range(cu[s], cu[s + 1]):
                    state.mul_(self.spec.decay).add_(u[t])
                    out[t] = state
            return (out @ self.w_out.T).to(x.dtype)

    @dataclasses.dataclass(frozen=True)
    class ToyConfig:
        width: int
        depth: int
        words: int
        decay: float
        eps: float
        heads: int
        inner: int

        @classmethod
        def from_dict(cls, d):
            r = KeyReader(d)
            return cls(r.integer("toy_width"), r.integer("toy_depth"), r.integer("toy_words"), r.number("toy_decay"),
                       r.number("toy_eps"), r.integer("toy_heads"), r.integer("toy_inner"))

    def plan(cfg):
        norm = RMSNormSpec(cfg.width, cfg.eps)
        layers = []
        for n in range(cfg.depth):
            p = f"toy.{n}."
            if n % 2 == 0:
                mixer = PartPlan("toy_decay", DecaySpec(cfg.width, cfg.decay), {"w_in": p + "in", "w_out": p + "out"})
            else:   # attention without position encoding, between the state layers
                mixer = PartPlan("attention", AttentionSpec(cfg.width, cfg.heads, 1, cfg.width // cfg.heads,
                                                            PartPlan("none", NoPositionSpec())),
                                 {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o"})
            layers.append(prenorm_layer(PartPlan("rmsnorm", norm, {"weight": p + "n1"}), mixer,
                                    PartPlan("rmsnorm", norm, {"weight": p + "n2"}),
                                    PartPlan("swiglu", SwiGLUSpec(cfg.width, cfg.inner),
                                             {"gate": p + "g", "up": p + "u", "down": p + "d"})))
        # layer 0 runs twice (two state blocks), and the last run reads the cache line of run 1
        schedule = [ScheduleEntry(n) for n in range(cfg.depth)] + [ScheduleEntry(0), ScheduleEntry(1, cache_of=1)]
        return ModelPlan("ToyDecayLM", cfg.words, cfg.width,
                         PartPlan("table", EmbeddingSpec(cfg.words, cfg.width), {"table": "toy.embed"}),
                         tuple(layers), tuple(schedule), PartPlan("rmsnorm", norm, {"weight": "toy.norm"}),
                         PartPlan("linear", HeadSpec(cfg.words, cfg.width), {"weight": "toy.embed"}), max_positions=512)

    register_architecture(Architecture("ToyDecayLM", ToyConfig, plan, description="test-only"))


TOY = {"architectures": ["ToyDecayLM"], "toy_width": 48, "toy_depth": 2, "toy_words": 90, "toy_decay": 0.8,
       "toy_eps": 1e-5, "toy_heads": 3, "toy_inner": 80}


def toy_plain(tensors, tokens):
    """The toy model on one whole sequence, float64, written out plainly."""
    t = {k: v for k, v in tensors.items()}
    h = P.embedding(t["toy.embed"], tokens)
    T = len(tokens)

    def decay_mixer(x, p):
        u = x @ t[p + "in"].T
        s = np.zeros(48)
        out = np.zeros_like(u)
        for i in range(T):
            s = 0.8 * s + u[i]
            out[i] = s
        return out @ t[p + "out"].T

    def attn(x, p, kv_from=None):
        kx = x if kv_from is None else kv_from
        q = (x @ t[p + "q"].T).reshape(T, 3, 16)
        k = (kx @ t[p + "k"].T).reshape(T, 1, 16)
        v = (kx @ t[p + "v"].T).reshape(T, 1, 16)
        o = np.zeros((T, 3, 16))
        for hh in range(3):
            s = q[:, hh] @ k[:, 0].T / 4.0
            s = np.where(np.triu(np.ones((T, T), bool), 1), -np.inf, s)
            o[:, hh] = P.softmax(s) @ v[:, 0]
        return o.reshape(T, 48) @ t[p + "o"].T

    def ffn(x, p):
        return P.feed_forward(x, t[p + "g"], t[p + "u"], t[p + "d"])

    runs = [(0, None), (1, None), (0, None), (1, "shared")]
    kv_input = None
    for layer, shared in runs:
        p = f"toy.{layer}."
        xn = P.rms_norm(h, t[p + "n1"], 1e-5)
        if layer == 0:
            a = decay_mixer(xn, p)
        elif shared is None:
            kv_input = xn
            a = attn(xn, p)
        else:
            a = attn(xn, p, kv_from=kv_input)        # keys and values of the earlier run
        h = h + a
        h = h + ffn(P.rms_norm(h, t[p + "n2"], 1e-5), p)
    return P.rms_norm(h, t["toy.norm"], 1e-5) @ t["toy.embed"].T


def test_toy_architecture_registers_builds_and_steps(tmp_path):
    import traces
    from burn_lm_b200 import Engine, write_random_model
    from tiny import random_tokens, row_error
    register_toy()
    folder = write_random_model(str(tmp_path / "toy"), TOY, seed=1, dtype="float32")
    cfg, tensors = P.read_model_folder(folder)
    reqs = {"a": random_tokens(1, 75, 90), "b": random_tokens(2, 20, 90), "c": random_tokens(3, 130, 90), "d": random_tokens(4, 9, 90)}
    want = {rid: toy_plain(tensors, toks) for rid, toks in reqs.items()}
    for what, steps in (("whole", traces.whole(reqs)), ("tail", traces.tail(reqs, 32)), ("batched", traces.batched(reqs, 2, [5, 32]))):
        eng = Engine.from_folder(folder, dtype="float32", max_tokens=traces.max_live_tokens(steps), max_seqs=2)
        kinds = [eng.cache.view(r).kind for r in range(4)]
        assert kinds == ["state", "kv", "state", "kv"] and not eng.cache.view(3).writes
        assert eng.cache.view(0).state.data_ptr() != eng.cache.view(2).state.data_ptr()
        got = traces.run_in_process(eng, steps, str(tmp_path / what), 90)
        for rid in reqs:
            err = row_error(got[rid], want[rid])
            assert err.max() < 1e-4, (what, rid, float(err.max()), int(err.argmax()))


# --------------------------------------------------------------------------------------------------
# a second toy: a feed-forward with routing and a position encoding added to the stream, both written
# here with torch operations and registered from here
# --------------------------------------------------------------------------------------------------
@dataclasses.dataclass(frozen=True)
class RoutedSpec:
    hidden_size: int
    inner: int
    experts: int


@dataclasses.dataclass(frozen=True)
class LearnedPositionSpec:
    hidden_size: int
    positions: int


def register_routed_toy():
    from burn_lm_b200 import register_architecture, register_part, Architecture, TensorSpec
    from burn_lm_b200.config import KeyReader
    from burn_lm_b200.parts import CacheNeed, Part, RMSNormSpec, AttentionSpec, NoPositionSpec, EmbeddingSpec, HeadSpec
    from burn_lm_b200.plan import ModelPlan, PartPlan, ScheduleEntry, prenorm_layer
    from burn_lm_b200 import registry

    if "ToyRoutedLM" in [a.name for a in registry.architectures()]:
        return

    @register_part("feed_forward", "toy_routed")
    class RoutedFeedForward(Part):
        """Every token goes to the expert with the largest router logit (fp32) and is weighted by that
        expert's softmax probability; an expert is a gated feed-forward."""
        family = "feed_forward"

        def tensor_specs(self):
            s, t = self.spec, self.tensor_names
            return [TensorSpec(t["router"], (s.experts, s.hidden_size), init="normal:0.5"),
                    TensorSpec(t["gate"], (s.experts * s.inner, s.hidden_size), init="normal:0.1"),
                    TensorSpec(t["up"], (s.experts * s.inner, s.hidden_size), init="normal:0.1"),
                    TensorSpec(t["down"], (s.experts * s.hidden_size, s.inner), init="normal:0.1")]

        def bind(self, loaded):
            s, t = self.spec, self.tensor_names
            self.router = loaded[t["router"]].float()
            self.gate = loaded[t["gate"]].float().view(s.experts, s.inner, s.hidden_size)
            self.up = loaded[t["up"]].float().view(s.experts, s.inner, s.hidden_size)
            self.down = loaded[t["down"]].float().view(s.experts, s.hidden_size, s.inner)

        def forward(self, x, step):
            xf = x.float()
            prob = torch.softmax(xf @ self.router.T, dim=-1)
            weight, expert = prob.max(dim=-1)
            out = torch.zeros_like(xf)
            for e in range(self.spec.experts):
                rows = (expert == e).nonzero().flatten()
                if rows.numel():
                    xe = xf[rows]
                    g = xe @ self.gate[e].T
                    out[rows] = ((g / (1 + torch.exp(-g))) * (xe @ self.up[e].T)) @ self.down[e].T * weight[rows, None]
            return out.to(x.dtype)

    @register_part("position", "toy_learned")
    class LearnedPosition(Part):
        """A stored vector per position, added to the stream after the embedding."""
        family = "position"

        def tensor_specs(self):
            return [TensorSpec(self.tensor_names["table"], (self.spec.positions, self.spec.hidden_size), init="normal:0.3")]

        def bind(self, loaded):
            self.table = loaded[self.tensor_names["table"]].float()

        def on_embedding(self, resid, step):
            resid += self.table[step.token_pos.long()]

    @dataclasses.dataclass(frozen=True)
    class RoutedConfig:
        width: int
        depth: int
        words: int
        experts: int
        inner: int
        heads: int
        positions: int

        @classmethod
        def from_dict(cls, d):
            r = KeyReader(d)
            return cls(r.integer("r_width"), r.integer("r_depth"), r.integer("r_words"), r.integer("r_experts"),
                       r.integer("r_inner"), r.integer("r_heads"), r.integer("r_positions"))

    def plan(cfg):
        norm = RMSNormSpec(cfg.width, 1e-6)
        layers = []
        for n in range(cfg.depth):
            p = f"r.{n}."
            layers.append(prenorm_layer(
                PartPlan("rmsnorm", norm, {"weight": p + "n1"}),
                PartPlan("attention", AttentionSpec(cfg.width, cfg.heads, cfg.heads, cfg.width // cfg.heads, PartPlan("none", NoPositionSpec())),
                         {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o"}),
                PartPlan("rmsnorm", norm, {"weight": p + "n2"}),
                PartPlan("toy_routed", RoutedSpec(cfg.width, cfg.inner, cfg.experts),
                         {"router": p + "router", "gate": p + "g", "up": p + "u", "down": p + "d"})))
        return ModelPlan("ToyRoutedLM", cfg.words, cfg.width,
                         PartPlan("table", EmbeddingSpec(cfg.words, cfg.width), {"table": "r.embed"}),
                         tuple(layers), tuple(ScheduleEntry(n) for n in range(cfg.depth)),
                         PartPlan("rmsnorm", norm, {"weight": "r.norm"}),
                         PartPlan("linear", HeadSpec(cfg.words, cfg.width), {"weight": "r.head"}), max_positions=cfg.positions,
                         stream_position=PartPlan("toy_learned", LearnedPositionSpec(cfg.width, cfg.positions), {"table": "r.pos"}))

    register_architecture(Architecture("ToyRoutedLM", RoutedConfig, plan, description="test-only"))


ROUTED = {"architectures": ["ToyRoutedLM"], "r_width": 64, "r_depth": 3, "r_words": 70, "r_experts": 5, "r_inner": 40,
          "r_heads": 2, "r_positions": 160}


def routed_plain(t, tokens):
    """The routed toy on one whole sequence, float64, written out plainly."""
    T = len(tokens)
    h = P.embedding(t["r.embed"], tokens) + t["r.pos"][:T]
    for n in range(3):
        p = f"r.{n}."
        xn = P.rms_norm(h, t[p + "n1"], 1e-6)
        q = (xn @ t[p + "q"].T).reshape(T, 2, 32)
        k = (xn @ t[p + "k"].T).reshape(T, 2, 32)
        v = (xn @ t[p + "v"].T).reshape(T, 2, 32)
        o = np.zeros((T, 2, 32))
        for hh in range(2):
            s = q[:, hh] @ k[:, hh].T / np.sqrt(32.0)
            s = np.where(np.triu(np.ones((T, T), bool), 1), -np.inf, s)
            o[:, hh] = P.softmax(s) @ v[:, hh]
        h = h + o.reshape(T, 64) @ t[p + "o"].T
        xn = P.rms_norm(h, t[p + "n2"], 1e-6)
        prob = P.softmax(xn @ t[p + "router"].T)
        out = np.zeros_like(xn)
        for i in range(T):
            e = int(prob[i].argmax())
            g = xn[i] @ t[p + "g"].reshape(5, 40, 64)[e].T
            u = xn[i] @ t[p + "u"].reshape(5, 40, 64)[e].T
            out[i] = ((g / (1 + np.exp(-g))) * u) @ t[p + "d"].reshape(5, 64, 40)[e].T * prob[i, e]
        h = h + out
    return P.rms_norm(h, t["r.norm"], 1e-6) @ t["r.head"].T


def test_toy_routed_feed_forward_and_stream_position(tmp_path):
    """A feed-forward with routing and a position encoding added to the stream, defined above, registered,
    built from a model folder and stepped whole, token by token and in unequal batches."""
    import traces
    from burn_lm_b200 import Engine, write_random_model
    from tiny import random_tokens, row_error
    register_routed_toy()
    folder = write_random_model(str(tmp_path / "routed"), ROUTED, seed=4, dtype="float32")
    cfg, tensors = P.read_model_folder(folder)
    reqs = {"a": random_tokens(5, 90, 70), "b": random_tokens(6, 33, 70), "c": random_tokens(7, 140, 70)}
    want = {rid: routed_plain(tensors, toks) for rid, toks in reqs.items()}
    used = set()
    for what, steps in (("whole", traces.whole(reqs)), ("tail", traces.tail(reqs, 32)), ("batched", traces.batched(reqs, 2, [5, 32]))):
        eng = Engine.from_folder(folder, dtype="float32", max_tokens=traces.max_live_tokens(steps), max_seqs=2)
        got = traces.run_in_process(eng, steps, str(tmp_path / what), 70)
        for rid in reqs:
            err = row_error(got[rid], want[rid])
            assert err.max() < 1e-4, (what, rid, float(err.max()), int(err.argmax()))
    # the router is not a constant: the first layer alone sends tokens to several experts
    t = tensors
    for rid, toks in reqs.items():
        h = P.embedding(t["r.embed"], toks) + t["r.pos"][: len(toks)]
        used |= set(P.softmax(P.rms_norm(h, t["r.0.n1"], 1e-6) @ t["r.0.router"].T).argmax(-1).tolist())
    assert len(used) >= 3


# --------------------------------------------------------------------------------------------------
# a third toy: the package's own parts, arranged so that the layers differ: attention over every key in
# the even layers, over a window of the latest keys in the odd ones (two cache groups)
# --------------------------------------------------------------------------------------------------
WINDOW = 24


def register_windowed_toy():
    from burn_lm_b200.architectures.llama import llama_plan
    from burn_lm_b200.config.llama import LlamaConfig
    from burn_lm_b200.registry import Architecture, architectures, register_architecture
    if "ToyWindowedLM" in [a.name for a in architectures()]:
        return

    def plan(cfg):
        base = llama_plan(cfg)
        layers = []
        for n, layer in enumerate(base.layers):
            if n % 2 == 1:
                mixer = layer.part("mixer")
                layer = layer.with_part("mixer", dataclasses.replace(mixer, spec=dataclasses.replace(mixer.spec, window=WINDOW)))
            layers.append(layer)
        return dataclasses.replace(base, architecture="ToyWindowedLM", layers=tuple(layers))

    register_architecture(Architecture(name="ToyWindowedLM", config_class=LlamaConfig, plan=plan,
                                       description="test only: full and windowed attention in turn"))


def windowed_plain(cfg, tensors, tokens):
    """The plain model with a window in the odd layers: one function per part, from tests/plain."""
    cfg = P.complete_config(cfg)
    inv_freq = P.model_inverse_frequencies(cfg)
    h = P.embedding(tensors["model.embed_tokens.weight"], tokens)
    for n in range(cfg["num_hidden_layers"]):
        lw = P.layer_weights(tensors, n)
        a = P.attention(P.rms_norm(h, lw["input_layernorm"], cfg["rms_norm_eps"]), lw["q_proj"], lw["k_proj"], lw["v_proj"],
                        lw["o_proj"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], inv_freq, "half",
                        window=WINDOW if n % 2 == 1 else None)
        h = h + a
        h = h + P.feed_forward(P.rms_norm(h, lw["post_attention_layernorm"], cfg["rms_norm_eps"]),
                               lw["gate_proj"], lw["up_proj"], lw["down_proj"])
    h = P.rms_norm(h, tensors["model.norm.weight"], cfg["rms_norm_eps"])
    return h @ tensors["model.embed_tokens.weight"].T


@pytest.mark.parametrize("dtype,tolerance", [("float32", 1e-4), ("bfloat16", 3e-2)])
def test_layers_with_and_without_a_window_in_one_model(tmp_path, dtype, tolerance):
    """Layers of one model that differ in their mixer's options: the windowed layers form a cache group of
    their own, and prompts, single tokens and batches of unequal lengths agree with the plain model; the
    window's edge is shown by comparing with the plain model without a window, which must differ."""
    import traces
    from burn_lm_b200 import Engine, write_random_model
    from tiny import random_tokens, row_error
    register_windowed_toy()
    cfg = {"architectures": ["ToyWindowedLM"], "model_type": "toy", "num_hidden_layers": 4, "hidden_size": 128,
           "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 192, "vocab_size": 300,
           "rope_theta": 10000.0, "rope_scaling": None, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
           "max_position_embeddings": 512, "hidden_act": "silu"}
    folder = write_random_model(str(tmp_path / "windowed"), cfg, seed=4, dtype="bfloat16")
    _, tensors = P.read_model_folder(folder)
    reqs = {"a": random_tokens(1, 150, 300), "b": random_tokens(2, 20, 300), "c": random_tokens(3, 70, 300), "d": random_tokens(4, WINDOW + 1, 300)}
    want = {rid: windowed_plain(cfg, tensors, toks) for rid, toks in reqs.items()}
    llama_like = dict(cfg, architectures=["LlamaForCausalLM"])
    without = P.forward(llama_like, tensors, reqs["a"])
    assert row_error(want["a"][WINDOW + 5:], without[WINDOW + 5:]).max() > 10 * tolerance      # the window matters
    assert row_error(want["a"][:WINDOW], without[:WINDOW]).max() < 1e-9                        # ... from its edge on
    for what, steps in (("whole", traces.whole(reqs)), ("tail", traces.tail(reqs, 32)), ("batched", traces.batched(reqs, 3, [5, 32]))):
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=traces.max_live_tokens(steps), max_seqs=3)
        tables = {eng.cache.view(r).block_table.data_ptr() for r in range(4)}
        assert len(tables) == 2 and eng.cache.view(1).window == WINDOW and not eng.cache.view(0).window
        got = traces.run_in_process(eng, steps, str(tmp_path / what), 300)
        for rid in reqs:
            err = row_error(got[rid], want[rid])
            assert err.max() < tolerance, (what, rid, float(err.max()), int(err.argmax()))
        eng.verify()


def test_windowed_layers_give_pages_back_while_sequences_grow(tmp_path):
    """Sequences of some hundred tokens on the model with a window of 24 keys in every other layer: the windowed
    group holds two or three pages a sequence however long it gets, the pages it gives back go to the other
    sequences of the batch and to the next batch, and every logit is still the plain model's (bfloat16, captured
    decode steps; prompts in two steps, then up to 200 single tokens, the shorter requests leaving earlier)."""
    import traces
    from burn_lm_b200 import Engine, write_random_model
    from tiny import random_tokens, row_error
    register_windowed_toy()
    cfg = {"architectures": ["ToyWindowedLM"], "model_type": "toy", "num_hidden_layers": 4, "hidden_size": 128,
           "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 192, "vocab_size": 300,
           "rope_theta": 10000.0, "rope_scaling": None, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
           "max_position_embeddings": 512, "hidden_act": "silu"}
    folder = write_random_model(str(tmp_path / "windowed_long"), cfg, seed=6, dtype="bfloat16")
    _, tensors = P.read_model_folder(folder)
    lengths = [500, 333, 260, 410, 129, 480]
    reqs = {f"r{n}": random_tokens(20 + n, length, 300) for n, length in enumerate(lengths)}
    steps = traces.batched(reqs, 3, [200, 60, 130], prompt_steps=2)
    eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=traces.max_live_tokens(steps), max_seqs=3)
    windowed = [g for g in eng.cache._kv_groups if g.need.window][0]
    most_held = 0
    real_reserve = eng.cache.reserve

    def watching(growth):
        nonlocal most_held
        real_reserve(growth)
        most_held = max(most_held, max(len(windowed.live_pages(s)) for s, _ in growth))
    eng.cache.reserve = watching
    got = traces.run_in_process(eng, steps, str(tmp_path / "o"), 300)
    eng.verify()
    assert max(windowed.dropped) == 0 and windowed.pages.free_count == eng.cache.n_pages      # all given back at the end
    # a prompt part of up to 150 tokens needs its own pages and those of the window before it; a decoding sequence two
    assert most_held <= 4
    for rid, toks in reqs.items():
        err = row_error(got[rid], windowed_plain(cfg, tensors, toks))
        assert err.max() < 3e-2, (rid, len(toks), float(err.max()), int(err.argmax()))


# --------------------------------------------------------------------------------------------------
# a fourth toy: another arrangement of a layer's parts.  One norm feeds the mixer and the feed-forward
# side by side, h = x + mixer(norm(x)) + feed_forward(norm(x)); every third layer has no feed-forward at
# all.  The block is written and registered here; the layer plans name other parts than the Llama
# decoder's pre-norm block does.
# --------------------------------------------------------------------------------------------------
def register_parallel_toy():
    from burn_lm_b200 import register_architecture, register_part, Architecture
    from burn_lm_b200.config.llama import LlamaConfig
    from burn_lm_b200.architectures.llama import llama_plan
    from burn_lm_b200.plan import LayerPlan, NamedPart
    from burn_lm_b200 import registry, kernels as K

    if "ToyParallelLM" in [a.name for a in registry.architectures()]:
        return

    @register_part("block", "toy_parallel")
    class ParallelBlock:
        family = "block"
        graph_safe = True

        def __init__(self, parts):
            assert set(parts) <= {"norm", "mixer", "feed_forward"} and {"norm", "mixer"} <= set(parts)
            self.norm, self.mixer, self.feed_forward = parts["norm"], parts["mixer"], parts.get("feed_forward")

        def forward(self, resid, delta, step, cache_view):
            x = self.norm.add_norm(resid, delta)              # adds the block before into the stream, then normalises
            a = self.mixer.forward(x, step, cache_view)
            if self.feed_forward is None:
                return a
            f = self.feed_forward.forward(x, step)
            if a.dtype == torch.float32:
                return a + f
            both = torch.empty_like(a, dtype=torch.float32)   # the two branches are summed in 32-bit
            K.convert(a, both)
            f32 = torch.empty_like(both)
            K.convert(f, f32)
            out = torch.empty_like(a)
            K.convert(both + f32, out)
            return out

    def plan(cfg):
        base = llama_plan(cfg)
        layers = []
        for n, layer in enumerate(base.layers):
            parts = [NamedPart("norm", "norm", layer.part("mixer_norm")), NamedPart("mixer", "mixer", layer.part("mixer"))]
            if n % 3 != 2:
                parts.append(NamedPart("feed_forward", "feed_forward", layer.part("feed_forward")))
            layers.append(LayerPlan("toy_parallel", tuple(parts)))
        return dataclasses.replace(base, architecture="ToyParallelLM", layers=tuple(layers),
                                   ignorable_tensors=base.ignorable_tensors)

    register_architecture(Architecture(name="ToyParallelLM", config_class=LlamaConfig, plan=plan,
                                       description="test only: one norm, mixer and feed-forward side by side"))


def parallel_plain(cfg, tensors, tokens):
    cfg = P.complete_config(cfg)
    inv_freq = P.model_inverse_frequencies(cfg)
    h = P.embedding(tensors["model.embed_tokens.weight"], tokens)
    for n in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{n}."
        x = P.rms_norm(h, tensors[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        a = P.attention(x, tensors[p + "self_attn.q_proj.weight"], tensors[p + "self_attn.k_proj.weight"],
                        tensors[p + "self_attn.v_proj.weight"], tensors[p + "self_attn.o_proj.weight"],
                        cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], inv_freq, "half")
        h = h + a
        if n % 3 != 2:
            h = h + P.feed_forward(x, tensors[p + "mlp.gate_proj.weight"], tensors[p + "mlp.up_proj.weight"], tensors[p + "mlp.down_proj.weight"])
    return P.rms_norm(h, tensors["model.norm.weight"], cfg["rms_norm_eps"]) @ tensors["model.embed_tokens.weight"].T


@pytest.mark.parametrize("dtype,tolerance", [("float32", 1e-4), ("bfloat16", 3e-2)])
def test_a_block_of_another_shape_is_a_plan_entry(tmp_path, dtype, tolerance):
    """A block with one shared norm, and layers without a feed-forward, registered from here: the model
    lists only the tensors those parts need, builds, and replays like any other."""
    import traces
    from burn_lm_b200 import Engine, write_random_model
    from burn_lm_b200.model import tensor_specs_of
    from tiny import random_tokens, row_error
    register_parallel_toy()
    cfg = {"architectures": ["ToyParallelLM"], "model_type": "toy", "num_hidden_layers": 3, "hidden_size": 128,
           "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 192, "vocab_size": 300,
           "rope_theta": 10000.0, "rope_scaling": None, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
           "max_position_embeddings": 512, "hidden_act": "silu"}
    names = {s.name for s in tensor_specs_of(cfg)}
    assert "model.layers.0.post_attention_layernorm.weight" not in names and "model.layers.2.mlp.down_proj.weight" not in names
    assert "model.layers.1.mlp.down_proj.weight" in names
    folder = write_random_model(str(tmp_path / "parallel"), cfg, seed=5, dtype="bfloat16")
    _, tensors = P.read_model_folder(folder)
    reqs = {"a": random_tokens(1, 150, 300), "b": random_tokens(2, 20, 300), "c": random_tokens(3, 70, 300)}
    want = {rid: parallel_plain(cfg, tensors, toks) for rid, toks in reqs.items()}
    for what, steps in (("whole", traces.whole(reqs)), ("tail", traces.tail(reqs, 32)), ("batched", traces.batched(reqs, 3, [5, 32, 9]))):
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=traces.max_live_tokens(steps), max_seqs=3)
        got = traces.run_in_process(eng, steps, str(tmp_path / what), 300)
        for rid in reqs:
            err = row_error(got[rid], want[rid])
            assert err.max() < tolerance, (what, rid, float(err.max()), int(err.argmax()))
        eng.verify()
