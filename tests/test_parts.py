"""Each part alone against the plain functions, and the generality the parts promise: a toy
mixer with state of its own (defined here) that is registered, built and stepped without a
change to the library; a run order that names a layer twice and shares a cache."""
import dataclasses
import json
import math

import numpy as np

import pytest
import torch

import plain_llama as pl
import trace_tools as tt
from conftest import TINY_B, require_gpu

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ctx():
    require_gpu()
    from hilbert_pruned_8b_b200.engine.workspace import Workspace
    from hilbert_pruned_8b_b200.kernels.ops import Ops
    from hilbert_pruned_8b_b200.parts import BuildContext

    def make(dtype):
        dev = torch.device(DEV)
        return BuildContext(device=dev, dtype=dtype, ops=Ops(dev), workspace=Workspace(dev), max_step_tokens=256)
    return make


def _step_for(ctx_, cache, lengths_before, new):
    from hilbert_pruned_8b_b200.engine.batch import StepEntry, build_step
    seqs = []
    for lb in lengths_before:
        s = cache.open()
        if lb:
            cache.reserve([(s, lb)])
            cache.commit(s, lb)
        seqs.append(s)
    entries = [StepEntry(s, [0] * n, []) for s, n in zip(seqs, new)]
    cache.reserve([(e.seq, e.seq.length + len(e.tokens)) for e in entries])
    return build_step(entries, cache, ctx_.workspace, ctx_.device), seqs


def _rel(a, b):
    return ((a.double().cpu() - b.double().cpu()).abs().max() / b.double().abs().max().clamp(min=1e-9)).item()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(ctx, dtype):
    from hilbert_pruned_8b_b200.config import PartSpec
    from hilbert_pruned_8b_b200.parts import NORMS
    c = ctx(dtype)
    norm = NORMS.build(PartSpec("rmsnorm", {"size": 200, "eps": 3e-6, "offset": 0.0}), c)
    assert [p.name for p in norm.params()] == ["weight"] and norm.params()[0].shape == (200,)
    w = torch.randn(200, device=DEV).to(torch.bfloat16)
    norm.bind({"weight": w})
    x = torch.randn(11, 200, device=DEV) * 5
    out = torch.empty(11, 200, device=DEV, dtype=dtype)
    norm.forward(x, out)
    ref = pl.rms_norm(x.double().cpu(), w.double().cpu(), 3e-6)
    assert _rel(out, ref) < (2e-6 if dtype == torch.float32 else 2 ** -8)


def test_rotary_part_matches_plain_frequencies_and_angles(ctx):
    from hilbert_pruned_8b_b200.config import PartSpec
    from hilbert_pruned_8b_b200.parts import POSITION_ENCODINGS
    import types
    c = ctx(torch.float32)
    llama3 = {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 32}
    rope = POSITION_ENCODINGS.build(PartSpec("rotary", {"head_dim": 48, "rotary_dim": 40, "theta": 500000.0,
                                                         "llama3": llama3}), c)
    want = pl.rope_inv_freq(40, 500000.0, llama3)
    assert (abs(rope.inv_freq_host - want) <= 1.2e-7 * want).all()
    pos = torch.tensor([0, 3, 200, 9000], dtype=torch.int32, device=DEV)
    step = types.SimpleNamespace(positions=pos, num_tokens=4, shared={})
    table, rot = rope.rotation_table(step)
    assert rot == 40 and rope.fusable
    ang = torch.from_numpy(rope.inv_freq_host)[None, :] * pos.cpu().float()[:, None]
    assert (table[..., 0].cpu().double() - torch.cos(ang.double())).abs().max() < 3e-7
    assert (table[..., 1].cpu().double() - torch.sin(ang.double())).abs().max() < 3e-7
    assert rope.rotation_table(step)[0] is table            # made once per step


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,window", [(6, 2, 48, None), (4, 1, 64, None), (4, 4, 16, 20)])
def test_attention_part_prefill_then_decode(ctx, dtype, nh, nkv, hd, window):
    """The mixer alone: a prompt in one step, then single tokens, against plain attention over
    the whole sequence; its output is ADDED to the residual."""
    from hilbert_pruned_8b_b200.cache import CacheManager
    from hilbert_pruned_8b_b200.config import PartSpec
    from hilbert_pruned_8b_b200.engine.batch import StepEntry, build_step
    from hilbert_pruned_8b_b200.parts import MIXERS
    c = ctx(dtype)
    H = 72
    rope = PartSpec("rotary", {"head_dim": hd, "rotary_dim": hd, "theta": 10000.0})
    mixer = MIXERS.build(PartSpec("attention", {"hidden_size": H, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd,
                                               "window": window, "position": rope}), c)
    torch.manual_seed(20)
    w = {p.name: (torch.randn(p.shape, device=DEV) / math.sqrt(p.shape[1])).to(torch.bfloat16) for p in mixer.params()}
    mixer.bind({k: v.to(dtype) for k, v in w.items()})
    cache = CacheManager({0: mixer.cache_need()}, {}, 512, c.device, dtype)
    T, P = 75, 70
    h = torch.randn(T, H, device=DEV).to(dtype)
    res0 = torch.randn(T, H, device=DEV)
    seq = cache.open()
    got = res0.clone()
    for lo, hi in [(0, P)] + [(t, t + 1) for t in range(P, T)]:
        e = [StepEntry(seq, [0] * (hi - lo), [])]
        cache.reserve([(seq, hi)])
        step = build_step(e, cache, c.workspace, c.device)
        mixer.forward(h[lo:hi].contiguous(), got[lo:hi], step, cache.view(0), None, True)
        cache.commit(seq, hi)
    rnd = (lambda x: x.float().to(torch.bfloat16).double()) if dtype == torch.bfloat16 else (lambda x: x)
    wd = {k: v.double().cpu() for k, v in w.items()}
    hd_ = h.double().cpu()
    q = rnd(pl.linear(hd_, wd["q_proj.weight"])).view(T, nh, hd)
    k = rnd(pl.linear(hd_, wd["k_proj.weight"])).view(T, nkv, hd)
    v = rnd(pl.linear(hd_, wd["v_proj.weight"])).view(T, nkv, hd)
    inv = pl.rope_inv_freq(hd, 10000.0, None)
    q, k = rnd(pl.rope(q, range(T), inv, hd)), rnd(pl.rope(k, range(T), inv, hd))
    a = rnd(pl.attention(q, k, v, window)).reshape(T, nh * hd)
    ref = res0.double().cpu() + pl.linear(a, wd["o_proj.weight"])
    assert _rel(got, ref) < (1e-5 if dtype == torch.float32 else 2e-2)
    cache.close(seq)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_embedding_and_head_parts(ctx, dtype):
    from hilbert_pruned_8b_b200.config import PartSpec
    from hilbert_pruned_8b_b200.parts import EMBEDDINGS, FEED_FORWARDS, HEADS
    import types
    c = ctx(dtype)
    torch.manual_seed(21)
    ffn = FEED_FORWARDS.build(PartSpec("swiglu", {"hidden_size": 72, "intermediate_size": 200}), c)
    w = {p.name: (torch.randn(p.shape, device=DEV) / math.sqrt(p.shape[1])).to(torch.bfloat16) for p in ffn.params()}
    ffn.bind({k: v.to(dtype) for k, v in w.items()})
    h = torch.randn(9, 72, device=DEV).to(dtype)
    res = torch.randn(9, 72, device=DEV)
    got = res.clone()
    ffn.forward(h, got, types.SimpleNamespace(num_tokens=9))
    rnd = (lambda x: x.float().to(torch.bfloat16).double()) if dtype == torch.bfloat16 else (lambda x: x)
    wd = {k: v.double().cpu() for k, v in w.items()}
    ref = res.double().cpu() + pl.swiglu(h.double().cpu(), wd["gate_proj.weight"], wd["up_proj.weight"],
                                         wd["down_proj.weight"], rnd)
    assert _rel(got, ref) < (1e-5 if dtype == torch.float32 else 2e-2)

    emb = EMBEDDINGS.build(PartSpec("embedding", {"vocab_size": 301, "hidden_size": 72}), c)
    table = torch.randn(301, 72, device=DEV).to(dtype)
    emb.bind({"weight": table})
    x = torch.empty(4, 72, device=DEV)
    emb.forward(torch.tensor([300, 0, 7, 7], dtype=torch.int32, device=DEV), x)
    assert torch.equal(x, table[[300, 0, 7, 7]].float())
    head = HEADS.build(PartSpec("lm_head", {"vocab_size": 301, "hidden_size": 72, "tied": True}), c)
    assert head.params()[0].optional and head.params()[0].absolute
    stored = head.tie(emb.weight)
    emb.share(stored)                                   # one copy of the table serves both
    emb.forward(torch.tensor([300, 0, 7, 7], dtype=torch.int32, device=DEV), x)
    assert torch.equal(x, table[[300, 0, 7, 7]].float())
    hn = torch.randn(4, 72, device=DEV).to(dtype)
    logits = torch.empty(4, 301, device=DEV)
    head.forward(hn, logits)
    assert _rel(logits, hn.double() @ table.double().t()) < (1e-5 if dtype == torch.float32 else 1e-5)


# --------------------------------------------------------------------------- a toy mixer with state
def _register_toy():
    """A mixer that keeps a decaying sum of its inputs per sequence (fixed-size state, no keys)
    and an architecture that alternates it with attention.  Everything is defined here."""
    from hilbert_pruned_8b_b200.config import (LayerSpec, LlamaConfig, ModelSpec, PartSpec, PlanEntry,
                                               register_architecture)
    from hilbert_pruned_8b_b200.parts import MIXERS, Mixer, ParamSpec, StateNeed

    @MIXERS.register("toy_decay")
    class ToyDecay(Mixer):
        graph_safe = False          # a Python loop over tokens: not something to capture in a graph

        def __init__(self, spec, ctx):
            super().__init__(spec, ctx)
            self.hidden, self.decay = spec.params["hidden_size"], spec.params["decay"]

        def params(self):
            return [ParamSpec("mix.weight", (self.hidden, self.hidden))]

        def bind(self, tensors):
            self.w = tensors["mix.weight"].float()

        def state_need(self):
            return StateNeed((self.hidden,), torch.float32)

        def forward(self, h, residual, step, cache, state, append):
            # tokens of a sequence in order; state[slot] carries over between steps
            t = 0
            slots = step.host_state_slots
            for b, n in enumerate(step.host_new):
                s = state[slots[b]]
                for i in range(n):
                    s.mul_(self.decay).add_(h[t].float())
                    residual[t] += s @ self.w.t()
                    t += 1

    class ToyConfig:
        architecture = "ToyHybridForCausalLM"
        model_type = "toy_hybrid"

        def __init__(self, base, decay):
            self.base, self.decay = base, decay

        @classmethod
        def from_dict(cls, root):
            return cls(LlamaConfig.from_dict({**root, "architectures": ["LlamaForCausalLM"]}), root["toy_decay"])

        def to_dict(self):
            return {**self.base.to_dict(), "architectures": [self.architecture], "model_type": self.model_type,
                    "toy_decay": self.decay}

        def model_spec(self):
            s = self.base.model_spec()
            toy = PartSpec("toy_decay", {"hidden_size": self.base.hidden_size, "decay": self.decay})
            layers = [ls.with_part("mixer", toy, prefix="toy.") if i % 2 == 0 else ls
                      for i, ls in enumerate(s.layers)]
            return dataclasses.replace(s, architecture=self.architecture, layers=layers)

    register_architecture(ToyConfig)
    return ToyConfig


class PlainToyHybrid(pl.PlainLlama):
    def __init__(self, folder, decay, round_to=None):
        super().__init__(folder, round_to=round_to)
        self.decay = decay

    def layer(self, x, i, positions):
        if i % 2:
            return super().layer(x, i, positions)
        c, w, p = self.cfg, self.w, f"{self.prefix}layers.{i}."
        h = self.rnd(pl.rms_norm(x, w[p + "input_layernorm.weight"], c["rms_norm_eps"]))
        s = torch.zeros(x.shape[1], dtype=x.dtype)
        rows = []
        for t in range(x.shape[0]):
            s = s * self.decay + h[t]
            rows.append(s @ w[p + "toy.mix.weight"].t())
        x = x + torch.stack(rows)
        h = self.rnd(pl.rms_norm(x, w[p + "post_attention_layernorm.weight"], c["rms_norm_eps"]))
        return x + pl.swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"],
                             self.rnd)


def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    require_gpu()
    import hilbert_pruned_8b_b200 as hb
    from hilbert_pruned_8b_b200.config import unregister_architecture
    from hilbert_pruned_8b_b200.engine.step import Engine
    from hilbert_pruned_8b_b200.parts import MIXERS
    ToyConfig = _register_toy()
    try:
        cfg = ToyConfig(hb.LlamaConfig.from_dict(TINY_B), 0.75)
        folder = hb.weights.write_random_model(str(tmp_path / "toy"), cfg, seed=31, fan_in_scale=1.0, norm_std=0.05)
        assert json.load(open(f"{folder}/config.json"))["architectures"] == ["ToyHybridForCausalLM"]
        eng = Engine.from_folder(folder, "float32", max_tokens=1024)
        assert sorted(eng.model.state_needs()) == [0, 2] and sorted(eng.model.cache_needs()) == [1]
        assert len(eng.cache.groups) == 1 and eng.cache.state_view(0).shape[1:] == (TINY_B["hidden_size"],)
        v = TINY_B["vocab_size"]
        reqs = {"p": tt.random_tokens(50, v, 900), "q": tt.random_tokens(21, v, 901), "r": tt.random_tokens(70, v, 902)}
        ref = tt.plain_logits(PlainToyHybrid(folder, 0.75), reqs)
        for make in (tt.trace_whole, lambda r: tt.trace_tail(r, 16),
                     lambda r: tt.trace_batches([{"p": (r["p"], 30), "q": (r["q"], 21)}, {"r": (r["r"], 5)}])):
            steps, _ = make(reqs)
            tt.compare(tt.run_in_process(eng, steps), ref, "float32", "toy hybrid")
        assert eng.cache.slots.num_held == 0
        # In bfloat16 the steps of few tokens fold the norms into the products around them where both
        # neighbours can: the toy mixer cannot (its block runs the norm kernels around it), the
        # attention layers between the toy layers can, and the two kinds hand over at every seam.
        eng16 = Engine.from_folder(folder, "bfloat16", max_tokens=1024)
        ops = eng16.ctx.ops
        ops.call_log = []
        steps, _ = tt.trace_tail(reqs, 16)
        got = tt.run_in_process(eng16, steps)
        log, ops.call_log = ops.call_log, None
        tt.compare(got, tt.plain_logits(PlainToyHybrid(folder, 0.75, round_to=torch.bfloat16), reqs), "bfloat16", "toy hybrid, folded norms")
        assert "hb_gemm_tc_fold" in log and "hb_rmsnorm" in log
    finally:
        unregister_architecture(ToyConfig)
        MIXERS.unregister("toy_decay")


# ------------------------------------------- a toy feed-forward with routing, another position encoding
def _register_toy_routed():
    """A feed-forward that routes every token to one of two small experts (router logits and
    the softmax in 32-bit, the chosen expert's output scaled by its probability), and a rotary
    position encoding with its own law of frequencies over half of each head.  Both are defined
    here, registered, and named by an architecture of their own; the library is not touched."""
    from hilbert_pruned_8b_b200.config import LlamaConfig, PartSpec, register_architecture
    from hilbert_pruned_8b_b200.parts import FEED_FORWARDS, POSITION_ENCODINGS, FeedForward, ParamSpec, PositionEncoding

    @FEED_FORWARDS.register("toy_top1")
    class ToyTop1(FeedForward):
        graph_safe = False          # plain torch operations that allocate

        def __init__(self, spec, ctx):
            super().__init__(spec, ctx)
            self.hidden, self.inner, self.experts = (int(spec.params[k]) for k in ("hidden_size", "inner_size", "experts"))

        def params(self):
            out = [ParamSpec("router.weight", (self.experts, self.hidden))]
            for e in range(self.experts):
                out += [ParamSpec(f"experts.{e}.in.weight", (self.inner, self.hidden)),
                        ParamSpec(f"experts.{e}.out.weight", (self.hidden, self.inner))]
            return out

        def bind(self, tensors):
            self.router = tensors["router.weight"].float()
            self.w_in = [tensors[f"experts.{e}.in.weight"].float() for e in range(self.experts)]
            self.w_out = [tensors[f"experts.{e}.out.weight"].float() for e in range(self.experts)]

        def forward(self, h, residual, step):
            x = h.float()
            prob = torch.softmax(x @ self.router.t(), dim=-1)
            top = prob.argmax(dim=-1)
            for e in range(self.experts):
                rows = (top == e).nonzero().flatten()
                if rows.numel():
                    y = torch.relu(x[rows] @ self.w_in[e].t()) @ self.w_out[e].t()
                    residual[rows] += y * prob[rows, e].unsqueeze(1)

    @POSITION_ENCODINGS.register("toy_linear_rotary")
    class ToyLinearRotary(PositionEncoding):
        graph_safe = False

        def __init__(self, spec, ctx):
            super().__init__(spec, ctx)
            self.rotary_dim = int(spec.params["rotary_dim"])
            self.slope = float(spec.params["slope"])

        def rotation_table(self, step):
            """([tokens, rot/2, 2] cosines and sines, rot): pair i turns by position * slope * (i + 1)."""
            key = f"toy_linear_rotary:{self.rotary_dim}:{self.slope}"
            if key not in step.shared:
                freq = self.slope * torch.arange(1, self.rotary_dim // 2 + 1, dtype=torch.float32, device=step.positions.device)
                ang = step.positions.float().unsqueeze(1) * freq.unsqueeze(0)
                step.shared[key] = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).contiguous()
            return step.shared[key], self.rotary_dim

    class ToyRoutedConfig:
        architecture = "ToyRoutedForCausalLM"
        model_type = "toy_routed"

        def __init__(self, base, slope):
            self.base, self.slope = base, slope

        @classmethod
        def from_dict(cls, root):
            return cls(LlamaConfig.from_dict({**root, "architectures": ["LlamaForCausalLM"]}), root["toy_slope"])

        def to_dict(self):
            return {**self.base.to_dict(), "architectures": [self.architecture], "model_type": self.model_type,
                    "toy_slope": self.slope}

        def model_spec(self):
            s, b = self.base.model_spec(), self.base
            pos = PartSpec("toy_linear_rotary", {"rotary_dim": b.head_dim // 2, "slope": self.slope})
            routed = PartSpec("toy_top1", {"hidden_size": b.hidden_size, "inner_size": 48, "experts": 2})
            layers = []
            for i, ls in enumerate(s.layers):
                mixer = PartSpec(ls.mixer.kind, {**ls.mixer.params, "position": pos})
                ls = ls.with_part("mixer", mixer)
                if i % 2:
                    ls = ls.with_part("feed_forward", routed, prefix="routed.")
                layers.append(ls)
            return dataclasses.replace(s, architecture=self.architecture, layers=layers)

    register_architecture(ToyRoutedConfig)
    return ToyRoutedConfig


class PlainToyRouted(pl.PlainLlama):
    def __init__(self, folder, slope):
        super().__init__(folder)
        hd = self.cfg["head_dim"]
        self.cfg["rotary_dim"] = hd // 2
        self.inv_freq = (np.float32(slope) * np.arange(1, hd // 4 + 1, dtype=np.float32)).astype(np.float32)

    def layer(self, x, i, positions):
        if i % 2 == 0:
            return super().layer(x, i, positions)
        c, w, p = self.cfg, self.w, f"{self.prefix}layers.{i}."
        nh, nkv, hd = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
        T = x.shape[0]
        h = pl.rms_norm(x, w[p + "input_layernorm.weight"], c["rms_norm_eps"])
        q = pl.rope(pl.linear(h, w[p + "self_attn.q_proj.weight"]).view(T, nh, hd), positions, self.inv_freq, c["rotary_dim"])
        k = pl.rope(pl.linear(h, w[p + "self_attn.k_proj.weight"]).view(T, nkv, hd), positions, self.inv_freq, c["rotary_dim"])
        v = pl.linear(h, w[p + "self_attn.v_proj.weight"]).view(T, nkv, hd)
        x = x + pl.linear(pl.attention(q, k, v).reshape(T, nh * hd), w[p + "self_attn.o_proj.weight"])
        h = pl.rms_norm(x, w[p + "post_attention_layernorm.weight"], c["rms_norm_eps"])
        prob = torch.softmax(h.float() @ w[p + "routed.router.weight"].float().t(), dim=-1).double()   # router in 32-bit
        rows = []
        for t in range(T):
            e = int(prob[t].argmax())
            y = torch.relu(h[t] @ w[p + f"routed.experts.{e}.in.weight"].t()) @ w[p + f"routed.experts.{e}.out.weight"].t()
            rows.append(y * prob[t, e])
        return x + torch.stack(rows)


def test_toy_routed_feed_forward_and_another_position_encoding(tmp_path):
    require_gpu()
    import hilbert_pruned_8b_b200 as hb
    from hilbert_pruned_8b_b200.config import unregister_architecture
    from hilbert_pruned_8b_b200.engine.step import Engine
    from hilbert_pruned_8b_b200.parts import FEED_FORWARDS, POSITION_ENCODINGS
    Cfg = _register_toy_routed()
    try:
        cfg = Cfg(hb.LlamaConfig.from_dict(TINY_B), 0.013)
        folder = hb.weights.write_random_model(str(tmp_path / "routed"), cfg, seed=41, fan_in_scale=1.0, norm_std=0.05)
        eng = Engine.from_folder(folder, "float32", max_tokens=1024)
        table = eng.model.weight_table()
        assert any(n.endswith("layers.1.routed.experts.1.out.weight") for n in table)
        assert not any("layers.1.mlp." in n for n in table) and any("layers.0.mlp.gate_proj.weight" in n for n in table)
        v = TINY_B["vocab_size"]
        reqs = {"p": tt.random_tokens(50, v, 920), "q": tt.random_tokens(21, v, 921), "r": tt.random_tokens(70, v, 922)}
        ref = tt.plain_logits(PlainToyRouted(folder, 0.013), reqs)
        for make in (tt.trace_whole, lambda r: tt.trace_tail(r, 16),
                     lambda r: tt.trace_batches([{"p": (r["p"], 30), "q": (r["q"], 21)}, {"r": (r["r"], 5)}])):
            steps, _ = make(reqs)
            tt.compare(tt.run_in_process(eng, steps), ref, "float32", "toy routed")
        assert min(eng.cache.pages_free()) == eng.cache.num_pages
    finally:
        unregister_architecture(Cfg)
        FEED_FORWARDS.unregister("toy_top1")
        POSITION_ENCODINGS.unregister("toy_linear_rotary")


# ------------------------------- a toy block with a post-norm, a position encoding that is no table
def _register_toy_postnorm():
    """A block of another shape (a norm BEHIND the mixer as well: ``x += post(mixer(pre(x)))``)
    with a role the library's block does not have, and a position encoding that is no table of
    half-split rotations (it turns the interleaved pairs (2i, 2i+1) itself).  Defined here,
    registered, named by an architecture of their own; the library is not touched."""
    from hilbert_pruned_8b_b200.config import LlamaConfig, PartSpec, register_architecture
    from hilbert_pruned_8b_b200.parts import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block,
                                              PositionEncoding)

    @BLOCKS.register("toy_postnorm")
    class ToyPostNormBlock(Block):
        ROLES = {"mixer_norm": NORMS, "mixer": MIXERS, "mixer_post_norm": NORMS, "feed_forward_norm": NORMS,
                 "feed_forward": FEED_FORWARDS}
        graph_safe = False

        def __init__(self, layer_spec, ctx):
            super().__init__(layer_spec, ctx)
            self.graph_safe = False         # torch operations that allocate

        def forward(self, x, step, cache, state, append):
            p = self.parts
            h = torch.empty(x.shape, dtype=self.ctx.dtype, device=x.device)
            p["mixer_norm"].forward(x, h)
            mixed = torch.zeros_like(x)                  # the mixer ADDS its output: into zeros here
            p["mixer"].forward(h, mixed, step, cache, state, append)
            post = torch.empty_like(x)
            p["mixer_post_norm"].forward(mixed, post)
            x += post
            p["feed_forward_norm"].forward(x, h)
            p["feed_forward"].forward(h, x, step)

    @POSITION_ENCODINGS.register("toy_interleaved")
    class ToyInterleaved(PositionEncoding):
        graph_safe = False

        def __init__(self, spec, ctx):
            super().__init__(spec, ctx)
            self.freq = float(spec.params["freq"])

        def apply(self, q, k, step):
            pos = step.positions.float()
            for x in (q, k):
                if x is None:
                    continue
                hd = x.shape[-1]
                ang = pos[:, None] * (self.freq * torch.arange(1, hd // 2 + 1, device=x.device, dtype=torch.float32))[None, :]
                cs, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
                a, b = x[..., 0::2].to(torch.float32, copy=True), x[..., 1::2].to(torch.float32, copy=True)
                x[..., 0::2] = (a * cs - b * sn).to(x.dtype)
                x[..., 1::2] = (b * cs + a * sn).to(x.dtype)

    class ToyPostNormConfig:
        architecture = "ToyPostNormForCausalLM"
        model_type = "toy_postnorm"

        def __init__(self, base, freq):
            self.base, self.freq = base, freq

        @classmethod
        def from_dict(cls, root):
            return cls(LlamaConfig.from_dict({**root, "architectures": ["LlamaForCausalLM"]}), root["toy_freq"])

        def to_dict(self):
            return {**self.base.to_dict(), "architectures": [self.architecture], "model_type": self.model_type,
                    "toy_freq": self.freq}

        def model_spec(self):
            s = self.base.model_spec()
            pos = PartSpec("toy_interleaved", {"freq": self.freq})
            layers = []
            for ls in s.layers:
                ls = ls.with_block("toy_postnorm").with_part("mixer", PartSpec(ls.mixer.kind, {**ls.mixer.params, "position": pos}))
                layers.append(ls.with_part("mixer_post_norm", ls.part("mixer_norm"), prefix="post_mixer_layernorm."))
            return dataclasses.replace(s, architecture=self.architecture, layers=layers)

    register_architecture(ToyPostNormConfig)
    return ToyPostNormConfig


class PlainToyPostNorm(pl.PlainLlama):
    def __init__(self, folder, freq):
        super().__init__(folder)
        self.freq = freq

    def turn(self, x, positions):
        hd = x.shape[-1]
        pos = torch.tensor(list(positions), dtype=torch.float32)
        ang = (pos[:, None] * (np.float32(self.freq) * torch.arange(1, hd // 2 + 1, dtype=torch.float32))[None, :]).double()
        cs, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        out = x.clone()
        out[..., 0::2] = x[..., 0::2] * cs - x[..., 1::2] * sn
        out[..., 1::2] = x[..., 1::2] * cs + x[..., 0::2] * sn
        return out

    def layer(self, x, i, positions):
        c, w, p = self.cfg, self.w, f"{self.prefix}layers.{i}."
        nh, nkv, hd = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
        T = x.shape[0]
        h = pl.rms_norm(x, w[p + "input_layernorm.weight"], c["rms_norm_eps"])
        q = self.turn(pl.linear(h, w[p + "self_attn.q_proj.weight"]).view(T, nh, hd), positions)
        k = self.turn(pl.linear(h, w[p + "self_attn.k_proj.weight"]).view(T, nkv, hd), positions)
        v = pl.linear(h, w[p + "self_attn.v_proj.weight"]).view(T, nkv, hd)
        mixed = pl.linear(pl.attention(q, k, v).reshape(T, nh * hd), w[p + "self_attn.o_proj.weight"])
        x = x + pl.rms_norm(mixed, w[p + "post_mixer_layernorm.weight"], c["rms_norm_eps"])
        h = pl.rms_norm(x, w[p + "post_attention_layernorm.weight"], c["rms_norm_eps"])
        return x + pl.swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"],
                             self.rnd)


def test_toy_block_with_a_post_norm_and_a_position_encoding_without_a_table(tmp_path):
    require_gpu()
    import hilbert_pruned_8b_b200 as hb
    from hilbert_pruned_8b_b200.config import unregister_architecture
    from hilbert_pruned_8b_b200.engine.step import Engine
    from hilbert_pruned_8b_b200.parts import BLOCKS, POSITION_ENCODINGS
    Cfg = _register_toy_postnorm()
    try:
        cfg = Cfg(hb.LlamaConfig.from_dict(TINY_B), 0.021)
        folder = hb.weights.write_random_model(str(tmp_path / "postnorm"), cfg, seed=51, fan_in_scale=1.0, norm_std=0.05)
        eng = Engine.from_folder(folder, "float32", max_tokens=1024)
        table = eng.model.weight_table()
        assert any(n.endswith("layers.2.post_mixer_layernorm.weight") for n in table)
        assert not eng.model.graph_safe
        v = TINY_B["vocab_size"]
        reqs = {"p": tt.random_tokens(50, v, 930), "q": tt.random_tokens(21, v, 931), "r": tt.random_tokens(70, v, 932)}
        ref = tt.plain_logits(PlainToyPostNorm(folder, 0.021), reqs)
        for make in (tt.trace_whole, lambda r: tt.trace_tail(r, 16),
                     lambda r: tt.trace_batches([{"p": (r["p"], 30), "q": (r["q"], 21)}, {"r": (r["r"], 5)}])):
            steps, _ = make(reqs)
            tt.compare(tt.run_in_process(eng, steps), ref, "float32", "toy post-norm")
        assert min(eng.cache.pages_free()) == eng.cache.num_pages
        # a part in a role the block does not have is refused by name
        bad = cfg.model_spec()
        bad = dataclasses.replace(bad, layers=[ls.with_block("prenorm") for ls in bad.layers])
        with pytest.raises(ValueError, match="mixer_post_norm"):
            Engine(bad, "float32", max_tokens=64)
    finally:
        unregister_architecture(Cfg)
        BLOCKS.unregister("toy_postnorm")
        POSITION_ENCODINGS.unregister("toy_interleaved")


# --------------------------------------------------------------------------- the run order is data
class PlainPlanned(pl.PlainLlama):
    """Plain model with a run order: (layer, cache_of) entries; an entry with cache_of reads the
    keys and values of that earlier entry and computes only its own queries."""

    def __init__(self, folder, plan):
        super().__init__(folder)
        self.plan = plan

    def hidden(self, tokens):
        c, w = self.cfg, self.w
        nh, nkv, hd = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
        x = pl.embed(tokens, w[self.prefix + "embed_tokens.weight"])
        T, pos, kv = len(tokens), list(range(len(tokens))), {}
        for idx, (layer, cache_of) in enumerate(self.plan):
            p = f"{self.prefix}layers.{layer}."
            h = pl.rms_norm(x, w[p + "input_layernorm.weight"], c["rms_norm_eps"])
            q = pl.rope(pl.linear(h, w[p + "self_attn.q_proj.weight"]).view(T, nh, hd), pos, self.inv_freq, c["rotary_dim"])
            if cache_of is None:
                k = pl.rope(pl.linear(h, w[p + "self_attn.k_proj.weight"]).view(T, nkv, hd), pos, self.inv_freq, c["rotary_dim"])
                kv[idx] = (k, pl.linear(h, w[p + "self_attn.v_proj.weight"]).view(T, nkv, hd))
            k, v = kv[idx if cache_of is None else cache_of]
            x = x + pl.linear(pl.attention(q, k, v).reshape(T, nh * hd), w[p + "self_attn.o_proj.weight"])
            h = pl.rms_norm(x, w[p + "post_attention_layernorm.weight"], c["rms_norm_eps"])
            x = x + pl.swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"],
                              self.rnd)
        return x


def test_run_order_names_a_layer_twice_and_shares_a_cache(model_folders):
    require_gpu()
    import hilbert_pruned_8b_b200 as hb
    from hilbert_pruned_8b_b200.config import PlanEntry
    from hilbert_pruned_8b_b200.engine.step import Engine
    from hilbert_pruned_8b_b200.weights import load_tensors
    folder = model_folders["strong_b"]
    plan = [(0, None), (1, None), (0, None), (2, 1), (1, 0)]
    spec = dataclasses.replace(hb.load_config(folder).model_spec(), plan=[PlanEntry(l, c) for l, c in plan])
    eng = Engine(spec, "float32", max_tokens=512)
    eng.model.bind(load_tensors(folder, eng.model.weight_table(), torch.float32, eng.device))
    eng._make_cache()
    assert sorted(eng.model.cache_needs()) == [0, 1, 2]            # entries 3 and 4 keep no keys of their own
    assert eng.cache.groups[0].k.shape[0] == 3
    reqs = {"u": tt.random_tokens(45, TINY_B["vocab_size"], 910), "w": tt.random_tokens(70, TINY_B["vocab_size"], 911)}
    ref = tt.plain_logits(PlainPlanned(folder, plan), reqs)
    for make in (tt.trace_whole, lambda r: tt.trace_tail(r, 20), lambda r: tt.trace_batches([{"u": (r["u"], 9), "w": (r["w"], 64)}])):
        steps, _ = make(reqs)
        tt.compare(tt.run_in_process(eng, steps), ref, "float32", "planned")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("model,window", [("strong_c", 40), ("strong_b", 70), ("strong_d", 64)])
def test_windowed_layers_give_pages_back_and_match_plain(model_folders, model, window, dtype):
    """Every layer with a window: the cache group frees pages that no later token can see
    (their page-table entries become -1) and the kernels mask the window's edge."""
    require_gpu()
    import hilbert_pruned_8b_b200 as hb
    from hilbert_pruned_8b_b200.config import PartSpec
    from hilbert_pruned_8b_b200.engine.step import Engine
    from hilbert_pruned_8b_b200.weights import load_tensors
    folder = model_folders[model]
    spec = hb.load_config(folder).model_spec()
    layers = [ls.with_part("mixer", PartSpec("attention", {**ls.mixer.params, "window": window})) for ls in spec.layers]
    spec = dataclasses.replace(spec, layers=layers)
    eng = Engine(spec, dtype, max_tokens=64 * 12)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    eng.model.bind(load_tensors(folder, eng.model.weight_table(), tdt, eng.device))
    eng._make_cache()
    vocab = spec.vocab_size
    reqs = {"a": tt.random_tokens(330, vocab, 920), "b": tt.random_tokens(150, vocab, 921)}
    plain = pl.PlainLlama(folder, round_to=torch.bfloat16 if dtype == "bfloat16" else None, window=window)
    ref = tt.plain_logits(plain, reqs)
    steps, _ = tt.trace_batches([{"a": (reqs["a"], 200), "b": (reqs["b"], 1)}])
    got = tt.run_in_process(eng, steps)
    tt.compare(got, ref, dtype, "windowed")
    # while "a" was 330 tokens long it held only the pages its window reaches, not all six
    seq = eng.open_sequence()
    eng.step_chunked([__import__("hilbert_pruned_8b_b200").engine.StepEntry(seq, reqs["a"][:300], [])])
    eng.step([__import__("hilbert_pruned_8b_b200").engine.StepEntry(seq, [reqs["a"][300]], [0])])
    held = [p for p in seq.pages[0] if p is not None]
    assert len(seq.pages[0]) == 5 and len(held) <= (window + 63) // 64 + 1
    eng.close_sequence(seq)
    assert min(eng.cache.pages_free()) == eng.cache.num_pages
