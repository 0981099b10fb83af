"""Plain, slow implementation of the Llama 3 dense decoder: the tests' oracle.

Whole sequences, no cache, no batching, one function per part, written from the
reference's formulas (``ct/`` = cleanroom-transformer/ of the reference; each function
cites file:line).  It shares no code with the library: it reads config.json with ``json``
and the weights with the ``safetensors`` package, and does its arithmetic in torch on the
CPU, by default in float64 (positions, frequencies and angles are float32 where the
reference computes them in float32, because that changes the numbers).

It was compared once with the reference's own CPU engine, built from source, on two tiny
models: see tests/golden/make_golden.py and tests/test_plain.py.

``round_to`` names the places where the bfloat16 serving path rounds activations
(norm output, projections, rotated q and k, cached v, attention output, activation
output); with ``round_to=torch.bfloat16`` the plain model rounds there too, so that the
comparison with the bfloat16 engine is about the kernels and not about the rounding points.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

F64 = torch.float64


# --------------------------------------------------------------------------- configuration
def read_config(model_dir: str) -> dict:
    """config.json keys as the reference reads them (ct/src/model.c:109-175, rope :36-58)."""
    with open(os.path.join(model_dir, "config.json")) as f:
        root = json.load(f)
    cfg = root.get("text_config") if isinstance(root.get("text_config"), dict) else root
    c = {k: int(cfg[k]) for k in ("hidden_size", "num_hidden_layers", "intermediate_size", "vocab_size",
                                  "num_attention_heads", "num_key_value_heads")}
    c["head_dim"] = int(cfg["head_dim"]) if cfg.get("head_dim") is not None else c["hidden_size"] // c["num_attention_heads"]
    c["rms_norm_eps"] = float(cfg.get("rms_norm_eps", 1e-6))
    rope = cfg.get("rope_parameters") if isinstance(cfg.get("rope_parameters"), dict) else cfg.get("rope_scaling")
    rope = rope if isinstance(rope, dict) else None
    theta = 10000.0
    if rope and "rope_theta" in rope:
        theta = float(rope["rope_theta"])
    elif "rope_theta" in cfg:
        theta = float(cfg["rope_theta"])
    partial = float((rope or {}).get("partial_rotary_factor", cfg.get("partial_rotary_factor", 1.0)))
    c["rope_theta"] = theta
    c["rotary_dim"] = int(c["head_dim"] * partial) & ~1
    rtype = (rope or {}).get("rope_type", (rope or {}).get("type"))
    c["llama3"] = None
    if rtype == "llama3":
        c["llama3"] = {k: float(rope[k]) for k in ("factor", "low_freq_factor", "high_freq_factor",
                                                   "original_max_position_embeddings")}
    c["tied"] = bool(cfg.get("tie_word_embeddings", root.get("tie_word_embeddings", False)))
    return c


class Widening(dict):
    """Tensors as stored; reading one widens it exactly to float64 (ct/src/model.c:259-270,291-307).
    Widening on use keeps a vocabulary-sized table at its stored size until it is needed."""

    def __getitem__(self, key):
        return super().__getitem__(key).to(F64)


def read_weights(model_dir: str, device: str = "cpu") -> Dict[str, torch.Tensor]:
    """Every tensor of model.safetensors; reads come back as float64."""
    from safetensors import safe_open
    out = Widening()
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            out[k] = f.get_tensor(k).to(device)
    return out


# --------------------------------------------------------------------------- parts
def rope_inv_freq(rotary_dim: int, theta: float, llama3: Optional[dict]) -> np.ndarray:
    """float32 inverse frequencies with llama3 scaling (ct/src/model.c:450-469)."""
    f32 = np.float32
    out = np.zeros(rotary_dim // 2, dtype=np.float32)
    for k in range(rotary_dim // 2):
        f = f32(1.0) / np.power(f32(theta), f32(2 * k) / f32(rotary_dim), dtype=np.float32)
        if llama3 is not None:
            pi = f32(3.14159265358979323846)
            factor, low, high = f32(llama3["factor"]), f32(llama3["low_freq_factor"]), f32(llama3["high_freq_factor"])
            ctx = f32(llama3["original_max_position_embeddings"])
            wavelen = f32(2.0) * pi / f
            low_wavelen, high_wavelen = ctx / low, ctx / high
            scaled = f / factor if wavelen > low_wavelen else f
            if not (wavelen < high_wavelen) and not (wavelen > low_wavelen):
                smooth = (ctx / wavelen - low) / (high - low)
                scaled = (f32(1.0) - smooth) * scaled / factor + smooth * scaled
            f = scaled
        out[k] = f32(f)
    return out


def embed(tokens: Sequence[int], table: torch.Tensor) -> torch.Tensor:
    """x[t] = E[token[t]], no scaling (ct/src/cpu_backend.c:236)."""
    return table[torch.as_tensor(list(tokens), dtype=torch.long, device=table.device)].clone()


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, offset: float = 0.0) -> torch.Tensor:
    """out = x / sqrt(mean(x^2) + eps) * (offset + w) (ct/src/cpu_backend.c:57-62)."""
    ss = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return x / torch.sqrt(ss + eps) * (offset + w)


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y[t][r] = sum_c x[t][c] W[r][c], W is [out, in] (ct/src/cpu_backend.c:39-54)."""
    return x @ w.t()


def rope(x: torch.Tensor, positions: Sequence[int], inv_freq: np.ndarray, rotary_dim: int) -> torch.Tensor:
    """Half-split rotation of x[T, heads, head_dim] (ct/src/cpu_backend.c:87-98): the angle is
    the float32 product inv_freq[i] * float(p); pairs are (i, i + rot/2); dims >= rot stay."""
    T = x.shape[0]
    half = rotary_dim // 2
    p = np.asarray(list(positions), dtype=np.float32)[:, None]
    ang = (inv_freq[None, :].astype(np.float32) * p).astype(np.float32)  # float32 product, as the reference
    ang = torch.from_numpy(ang.astype(np.float64)).to(x.device)
    cs, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    x1, x2 = x[..., :half], x[..., half:rotary_dim]
    out[..., :half] = x1 * cs - x2 * sn
    out[..., half:rotary_dim] = x2 * cs + x1 * sn
    assert out.shape[0] == T
    return out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: Optional[int] = None) -> torch.Tensor:
    """Causal grouped-query attention of one whole sequence (ct/src/cpu_backend.c:102-124):
    q[T, nh, hd], k,v[T, nkv, hd]; head j reads kv head j // (nh/nkv); scores q.k / sqrt(hd)
    over keys 0..t (only the last ``window`` if given), max-subtracted softmax, weighted sum."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    scale = 1.0 / math.sqrt(float(hd))
    out = torch.zeros(T, nh, hd, dtype=q.dtype, device=q.device)
    for j in range(nh):
        g = j // group
        sc = (q[:, j, :] @ k[:, g, :].t()) * scale                      # [T, T]
        t_idx = torch.arange(T, device=q.device)
        mask = t_idx[None, :] > t_idx[:, None]
        if window is not None:
            mask = mask | (t_idx[None, :] < (t_idx[:, None] - window + 1))
        sc = sc.masked_fill(mask, float("-inf"))
        sc = sc - sc.max(dim=-1, keepdim=True).values
        e = torch.exp(sc)
        pr = e / e.sum(dim=-1, keepdim=True)
        out[:, j, :] = pr @ v[:, g, :]
    return out


def silu(z: torch.Tensor) -> torch.Tensor:
    """z / (1 + exp(-z)) (ct/src/ops_common.h:56)."""
    return z / (1.0 + torch.exp(-z))


def swiglu(h: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor, rnd) -> torch.Tensor:
    """(silu(h Wg^T) * (h Wu^T)) Wd^T (ct/src/cpu_backend.c:248-251)."""
    a = rnd(silu(linear(h, wg)) * linear(h, wu))
    return linear(a, wd)


# --------------------------------------------------------------------------- the model
class PlainLlama:
    def __init__(self, model_dir: str, round_to: Optional[torch.dtype] = None, window: Optional[int] = None,
                 device: str = "cpu"):
        """``device``: where torch does the arithmetic.  The CPU by default; the models with a full
        vocabulary and real layer widths run the same float64 operations on the GPU, where they
        take seconds instead of minutes."""
        self.cfg = read_config(model_dir)
        self.w = read_weights(model_dir, device)
        self.prefix = "model.language_model." if "model.language_model.embed_tokens.weight" in self.w else "model."
        self.inv_freq = rope_inv_freq(self.cfg["rotary_dim"], self.cfg["rope_theta"], self.cfg["llama3"])
        self.round_to = round_to
        self.window = window

    def rnd(self, x: torch.Tensor) -> torch.Tensor:
        return x if self.round_to is None else x.to(torch.float32).to(self.round_to).to(F64)

    def layer(self, x: torch.Tensor, i: int, positions: Sequence[int]) -> torch.Tensor:
        """x += Attn(N(x)); x += MLP(N(x)) (ct/src/cpu_backend.c:237-252)."""
        c, w, p = self.cfg, self.w, f"{self.prefix}layers.{i}."
        nh, nkv, hd = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
        T = x.shape[0]
        h = self.rnd(rms_norm(x, w[p + "input_layernorm.weight"], c["rms_norm_eps"]))
        q = self.rnd(linear(h, w[p + "self_attn.q_proj.weight"])).view(T, nh, hd)
        k = self.rnd(linear(h, w[p + "self_attn.k_proj.weight"])).view(T, nkv, hd)
        v = self.rnd(linear(h, w[p + "self_attn.v_proj.weight"])).view(T, nkv, hd)
        q = self.rnd(rope(q, positions, self.inv_freq, c["rotary_dim"]))
        k = self.rnd(rope(k, positions, self.inv_freq, c["rotary_dim"]))
        a = self.rnd(attention(q, k, v, self.window)).reshape(T, nh * hd)
        x = x + linear(a, w[p + "self_attn.o_proj.weight"])
        h = self.rnd(rms_norm(x, w[p + "post_attention_layernorm.weight"], c["rms_norm_eps"]))
        x = x + swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"],
                       self.rnd)
        return x

    def hidden(self, tokens: Sequence[int]) -> torch.Tensor:
        table = dict.__getitem__(self.w, self.prefix + "embed_tokens.weight")      # rows are widened after the gather
        x = embed(tokens, table).to(F64)
        positions = list(range(len(tokens)))
        for i in range(self.cfg["num_hidden_layers"]):
            x = self.layer(x, i, positions)
        return x

    def logits_at(self, tokens: Sequence[int], places: Sequence[int]) -> torch.Tensor:
        """Logits at the given positions only: [len(places), vocab] float64."""
        x = self.hidden(tokens)[torch.as_tensor(list(places), dtype=torch.long, device=self.hidden_device())]
        h = self.rnd(rms_norm(x, self.w[self.prefix + "norm.weight"], self.cfg["rms_norm_eps"]))
        head = self.w[self.prefix + "embed_tokens.weight"] if self.cfg["tied"] else self.w["lm_head.weight"]
        return linear(h, head)

    def hidden_device(self):
        return dict.__getitem__(self.w, self.prefix + "norm.weight").device

    def logits(self, tokens: Sequence[int]) -> torch.Tensor:
        """Logits at every position of one whole sequence: [T, vocab] float64.  The reference
        normalises and reads out the last position only (ct/src/cpu_backend.c:253-259); a
        position's logits depend on earlier tokens only, so every prefix is read out here."""
        x = self.hidden(tokens)
        h = self.rnd(rms_norm(x, self.w[self.prefix + "norm.weight"], self.cfg["rms_norm_eps"]))
        head = self.w[self.prefix + "embed_tokens.weight"] if self.cfg["tied"] else self.w["lm_head.weight"]
        return linear(h, head)


# --------------------------------------------------------------------------- sampling
def greedy(logits: torch.Tensor) -> int:
    """Largest logit, lowest index on ties."""
    m = logits.max()
    return int(torch.nonzero(logits == m)[0, 0])


def temperature_probs(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """softmax(logits / temperature), max-subtracted, in float64."""
    z = logits.to(F64) / temperature
    e = torch.exp(z - z.max())
    return e / e.sum()


def inverse_cdf(probs: torch.Tensor, u: float) -> int:
    """The first index whose cumulative probability exceeds u."""
    c = torch.cumsum(probs, 0)
    idx = int(torch.searchsorted(c, torch.tensor(u, dtype=c.dtype), right=True))
    return min(idx, probs.numel() - 1)


def generate_greedy(model: PlainLlama, prompt: Sequence[int], max_new: int, stop: Sequence[int] = ()) -> List[int]:
    toks = list(prompt)
    out: List[int] = []
    for _ in range(max_new):
        nxt = greedy(model.logits(toks)[-1])
        out.append(nxt)
        toks.append(nxt)
        if nxt in stop:
            break
    return out
