"""The plain implementation itself (no GPU): against the reference engine's stored logits,
and each of its parts against an independent statement of the same formula."""
import json
import math
import os
import sys

import numpy as np
import pytest
import torch

import plain_llama as pl

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
from golden_models import GOLDEN_MODELS, golden_tokens, write_golden_model  # noqa: E402


@pytest.fixture(scope="module")
def golden(tmp_path_factory):
    out = {}
    for name, spec in GOLDEN_MODELS.items():
        d = str(tmp_path_factory.mktemp(name))
        write_golden_model(d, spec)
        out[name] = (pl.PlainLlama(d), golden_tokens(spec), d)
    return out


def test_plain_equals_the_reference_engine(golden):
    """Logits of the reference's CPU engine (built from its source, see golden/make_golden.py)
    on two tiny models: float32 engine against float64 plain, the reference's own parity
    bound 1e-4 * max(1, |logit|) (cleanroom-transformer/tools/parity.py:171-190)."""
    with open(os.path.join(HERE, "golden", "reference_logits.json")) as f:
        cases = json.load(f)["cases"]
    assert len(cases) == 16
    for c in cases:
        model, toks, _ = golden[c["model"]]
        lg = model.logits(toks[: c["n_tokens"]])[-1][c["ids"]]
        ref = torch.tensor(c["logits"], dtype=torch.float64)
        assert ((lg - ref).abs() / ref.abs().clamp(min=1.0)).max() < 1e-4
        assert (lg - ref).abs().max() < 2e-5


def test_prefix_property(golden):
    """A position's logits depend on earlier tokens only."""
    model, toks, _ = golden["golden_b"]
    full = model.logits(toks[:20])
    assert torch.allclose(full[:9], model.logits(toks[:9]), atol=1e-12)


def test_rope_frequencies_llama3_bands():
    f = pl.rope_inv_freq(32, 500000.0, None)
    assert f[0] == 1.0 and f.dtype == np.float32 and np.all(np.diff(f) < 0)
    s = pl.rope_inv_freq(32, 500000.0, {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                        "original_max_position_embeddings": 32})
    wavelen = 2 * math.pi / f
    high, low = 32 / 4.0, 32 / 1.0
    assert np.array_equal(s[wavelen < high], f[wavelen < high])                # short waves kept
    assert np.allclose(s[wavelen > low], f[wavelen > low] / 8.0, rtol=1e-6)    # long waves divided
    mid = (wavelen >= high) & (wavelen <= low)
    assert mid.any() and np.all(s[mid] <= f[mid] * (1 + 1e-6)) and np.all(s[mid] >= f[mid] / 8.0 * (1 - 1e-6))


def test_rope_is_a_rotation_of_half_split_pairs():
    x = torch.randn(3, 2, 8, dtype=torch.float64)
    inv = pl.rope_inv_freq(6, 10000.0, None)
    y = pl.rope(x, [0, 5, 9], inv, 6)
    assert torch.equal(y[0], x[0])                                   # position 0: identity
    assert torch.equal(y[..., 6:], x[..., 6:])                       # beyond the rotary dims
    assert torch.allclose(y[..., :6].norm(dim=-1), x[..., :6].norm(dim=-1))
    a = float(np.float32(inv[1]) * np.float32(5))
    assert abs(y[1, 0, 1] - (x[1, 0, 1] * math.cos(a) - x[1, 0, 4] * math.sin(a))) < 1e-12
    assert abs(y[1, 0, 4] - (x[1, 0, 4] * math.cos(a) + x[1, 0, 1] * math.sin(a))) < 1e-12


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    q, k, v = (torch.randn(6, 4, 8, dtype=torch.float64), torch.randn(6, 2, 8, dtype=torch.float64),
               torch.randn(6, 2, 8, dtype=torch.float64))
    out = pl.attention(q, k, v)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])     # first token, groups of 2
    sc = (q[4, 2] @ k[:5, 1].t()) / math.sqrt(8.0)
    assert torch.allclose(out[4, 2], torch.softmax(sc, 0) @ v[:5, 1])
    w = pl.attention(q, k, v, window=2)
    sc = (q[4, 2] @ k[3:5, 1].t()) / math.sqrt(8.0)
    assert torch.allclose(w[4, 2], torch.softmax(sc, 0) @ v[3:5, 1])


def test_norm_and_swiglu():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    y = pl.rms_norm(x, w, 1e-5)
    inv = 1 / math.sqrt(12.5 + 1e-5)
    assert torch.allclose(y, torch.tensor([[3 * inv * 2, 4 * inv * 0.5]], dtype=torch.float64))
    assert torch.allclose(pl.rms_norm(x, w, 1e-5, offset=1.0), x * inv * (1 + w))
    z = torch.tensor([-2.0, 0.0, 1.5], dtype=torch.float64)
    assert torch.allclose(pl.silu(z), z * torch.sigmoid(z))


def test_sampling_reference():
    lg = torch.tensor([0.1, 2.0, 2.0, -1.0])
    assert pl.greedy(lg) == 1
    p = pl.temperature_probs(lg, 0.5)
    assert abs(p.sum() - 1) < 1e-12 and p[1] == p[2] > p[0]
    assert pl.inverse_cdf(p, 0.0) == 0 and pl.inverse_cdf(p, float(p[0]) + 1e-9) == 1
    assert pl.inverse_cdf(p, 0.999999) == 3


def test_rounding_option_changes_little_but_something(golden):
    _, toks, d = golden["golden_a"]
    a = pl.PlainLlama(d).logits(toks[:12])
    b = pl.PlainLlama(d, round_to=torch.bfloat16).logits(toks[:12])
    err = (a - b).abs().max().item()
    assert 0 < err < 0.05 * a.abs().max().item()
