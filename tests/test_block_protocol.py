"""The block's decisions about folding norms into the products around them, with fake parts on the
CPU: who is asked to prepare what, when the norm kernels run, and that parts which do not take part
are called exactly as before."""
import types

import torch

from hilbert_pruned_8b_b200.config.spec import LayerSpec, PartSpec
from hilbert_pruned_8b_b200.parts import FEED_FORWARDS, MIXERS, NORMS, FeedForward, Mixer, Norm
from hilbert_pruned_8b_b200.parts.base import BuildContext
from hilbert_pruned_8b_b200.parts.block import PreNormBlock

LOG = []


class _Workspace:
    def __init__(self):
        self.buffers = {}

    def buffer(self, name, shape, dtype):
        key = (name, tuple(shape), dtype)
        if key not in self.buffers:
            self.buffers[key] = torch.zeros(shape, dtype=dtype)
        return self.buffers[key]


class _Ops:
    def __init__(self, limit):
        self.limit = limit

    def can_fold_norm(self, tokens, size, dtype):
        return tokens <= self.limit


def _register():
    @NORMS.register("fake_norm")
    class FakeNorm(Norm):
        def __init__(self, spec, ctx):
            super().__init__(spec, ctx)
            self.size, self.name = spec.params["size"], spec.params["name"]

        def forward(self, x, out, rows=None):
            LOG.append(("norm", self.name))

        def fold_request(self, out):
            return ("request", self.name, out)

    @MIXERS.register("fake_folding_mixer")
    class FoldingMixer(Mixer):
        folds_norms = True

        def forward(self, h, residual, step, cache, state, append, prepared=None, prepare=None):
            LOG.append(("mixer", prepared, prepare[:2] if prepare else None))
            return ("prepared-by-mixer", prepare[1]) if prepare else None

    @MIXERS.register("fake_plain_mixer")
    class PlainMixer(Mixer):
        def forward(self, h, residual, step, cache, state, append):
            LOG.append(("plain mixer",))

    @FEED_FORWARDS.register("fake_folding_ff")
    class FoldingFF(FeedForward):
        folds_norms = True

        def forward(self, h, residual, step, prepared=None, prepare=None):
            LOG.append(("ff", prepared, prepare[:2] if prepare else None))
            return ("prepared-by-ff", prepare[1]) if prepare else None

    @FEED_FORWARDS.register("fake_plain_ff")
    class PlainFF(FeedForward):
        def forward(self, h, residual, step):
            LOG.append(("plain ff",))


def _unregister():
    NORMS.unregister("fake_norm")
    for n in ("fake_folding_mixer", "fake_plain_mixer"):
        MIXERS.unregister(n)
    for n in ("fake_folding_ff", "fake_plain_ff"):
        FEED_FORWARDS.unregister(n)


def _block(mixer, ff, limit=16):
    ctx = BuildContext(torch.device("cpu"), torch.bfloat16, _Ops(limit), _Workspace(), 64)
    parts = {"mixer_norm": PartSpec("fake_norm", {"size": 32, "name": "a"}), "mixer": PartSpec(mixer, {}),
             "feed_forward_norm": PartSpec("fake_norm", {"size": 32, "name": "b"}), "feed_forward": PartSpec(ff, {})}
    spec = LayerSpec("layers.0.", parts, {r: "" for r in parts})
    return PreNormBlock(spec, ctx)


def _step(tokens):
    return types.SimpleNamespace(num_tokens=tokens)


def test_block_folds_only_where_both_neighbours_can():
    _register()
    try:
        x = torch.zeros(4, 32)
        # both parts fold, few tokens, nobody in front prepared, the next block asks
        LOG.clear()
        blk = _block("fake_folding_mixer", "fake_folding_ff")
        assert blk.fold_request(_step(4))[:2] == ("request", "a")
        out = blk.forward(x, _step(4), None, None, True, prepared=None, prepare_next=("request", "next", None))
        assert LOG == [("norm", "a"), ("mixer", None, ("request", "b")), ("ff", ("prepared-by-mixer", "b"), ("request", "next"))]
        assert out == ("prepared-by-ff", "next")
        # the block in front prepared this block's first norm: no norm kernel at all
        LOG.clear()
        blk.forward(x, _step(4), None, None, True, prepared=("prepared-by-ff", "a"), prepare_next=None)
        assert LOG == [("mixer", ("prepared-by-ff", "a"), ("request", "b")), ("ff", ("prepared-by-mixer", "b"), None)]
        # many tokens: nothing is asked for, both norms run, nothing is handed on
        LOG.clear()
        assert blk.fold_request(_step(40)) is None
        out = blk.forward(x, _step(40), None, None, True, prepared=None, prepare_next=("request", "next", None))
        assert LOG == [("norm", "a"), ("mixer", None, None), ("norm", "b"), ("ff", None, None)] and out is None
        # a feed-forward that does not take part: the mixer is not asked to prepare, the norm in front of it runs
        LOG.clear()
        blk = _block("fake_folding_mixer", "fake_plain_ff")
        out = blk.forward(x, _step(4), None, None, True, prepared=None, prepare_next=("request", "next", None))
        assert LOG == [("norm", "a"), ("mixer", None, None), ("norm", "b"), ("plain ff",)] and out is None
        # a mixer that does not take part: the block asks nobody in front, runs its norms, and the
        # feed-forward still prepares the next block's norm
        LOG.clear()
        blk = _block("fake_plain_mixer", "fake_folding_ff")
        assert blk.fold_request(_step(4)) is None
        out = blk.forward(x, _step(4), None, None, True, prepared=None, prepare_next=("request", "next", None))
        assert LOG == [("norm", "a"), ("plain mixer",), ("norm", "b"), ("ff", None, ("request", "next"))]
        assert out == ("prepared-by-ff", "next")
        # a product that could not prepare (returns None): the norm runs
        LOG.clear()
        blk = _block("fake_folding_mixer", "fake_folding_ff", limit=16)
        blk.mixer.forward = lambda h, r, s, c, st, ap, prepared=None, prepare=None: LOG.append(("mixer declined",))
        blk.forward(x, _step(4), None, None, True)
        assert LOG == [("norm", "a"), ("mixer declined",), ("norm", "b"), ("ff", None, None)]
    finally:
        _unregister()
