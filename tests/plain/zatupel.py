"""Whole-sequence Zatupel decoder, written from the design's equations: one request, all of its tokens, every
time; no cache, no state carried, no batching, no fusing.  float64 on the CPU by default, so the oracle's own
rounding is far below the tolerances of the engine under test.  One function per mechanism.

Notation: T tokens, W model width, H query heads, G key/value heads, D query/key size of a head, E value size
of a head, N heads of a recurrent mixer with K channels each.
"""
import json
import math
import os

import torch

from .safetensors_reader import read_safetensors


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last dimension (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return rms_unit(x, eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gated_gelu(x, w_gate, w_up, w_down):
    """down( gelu_tanh(gate x) * (up x) )."""
    return (gelu_tanh(x @ w_gate.t()) * (x @ w_up.t())) @ w_down.t()


def rotate_neighbours(x, positions, base, dims):
    """Rotary encoding of x[T, heads, D] on its first ``dims`` channels, channel 2i paired with 2i+1;
    angle = position * base^(-2i/dims).  The other channels pass unchanged."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=x.dtype)
    freq = torch.pow(torch.tensor(float(base), dtype=x.dtype), -2.0 * i / dims)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def visible(T, size, keep_first):
    """mask[i, j]: query i sees key j if j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def mixed_head_attention(q, k, v, scale, size, keep_first, talk):
    """q[T,H,D], k[T,G,D], v[T,G,E].  Each head's softmax over its visible keys; then the heads' weights are mixed,
    weight_h <- sum_g talk[h,g] weight_g; head h applies its mixed weights to the values of kv head h // (H/G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    mask = visible(T, size, keep_first)
    weights = []
    for h in range(H):
        s = (q[:, h] @ k[:, h // (H // G)].t()) * scale
        weights.append(torch.softmax(s.masked_fill(~mask, float("-inf")), dim=-1))
    weights = torch.stack(weights)                                   # [H, T, T]
    mixed = torch.einsum("hg,gij->hij", talk, weights)
    return torch.stack([mixed[h] @ v[:, h // (H // G)] for h in range(H)], dim=1)     # [T, H, E]


def attention_mixer(x, positions, w, m, v_first):
    """The attention mixer on x[T,W] (its normed input).  ``w``: the mixer's tensors by short name; ``m``: its
    configuration.  ``v_first``: the values of the first value-mixing layer (None in that layer and in layers that
    do not mix).  Returns (output [T,W], the values that this layer keeps)."""
    T = x.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (x @ w["q"].t()).view(T, H, D)
    k = (x @ w["k"].t()).view(T, G, D)
    v = (x @ w["v"].t()).view(T, G, E)
    q = rotate_neighbours(q, positions, m["rot"]["base"], m["rot"]["dims"])
    k = rotate_neighbours(k, positions, m["rot"]["base"], m["rot"]["dims"])
    if v_first is not None:
        lam = w["vmix"]
        v = (1.0 - lam) * v + lam * v_first
    o = mixed_head_attention(q, k, v, m["scale"], m["mask"]["size"], m["mask"]["keep_first"], w["talk"])
    gate = torch.sigmoid(x @ w["g"].t())                             # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * E) @ w["o"].t(), v


def _head_finish(o, norm_w, gate, w_o, eps):
    """o[T,N,K]: every head divided by its root mean square, heads side by side, times the weight, times the gate,
    then the output projection."""
    T = o.shape[0]
    return ((rms_unit(o, eps).reshape(T, -1) * norm_w) * gate) @ w_o.t()


def wkv_mixer(x, w, m, eps):
    """Time mixing with a shifted input, a decay that depends on the input, and a bonus for the current token.
    S is [K, K] per head (key channel x value channel), zero before the first token."""
    T = x.shape[0]
    N, K = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros_like(x[:1]), x[:-1]], dim=0)
    mix = {s: x + (prev - x) * w["mu." + s] for s in "rkvgw"}
    r = (mix["r"] @ w["r"].t()).view(T, N, K)
    k = (mix["k"] @ w["k"].t()).view(T, N, K)
    v = (mix["v"] @ w["v"].t()).view(T, N, K)
    g = mix["g"] @ w["g"].t()
    gate = g * torch.sigmoid(g)
    decay = torch.exp(-torch.exp(torch.tanh(mix["w"] @ w["w1"].t()) @ w["w2"].t() + w["w0"])).view(T, N, K)
    u = w["u"]
    S = torch.zeros(N, K, K, dtype=x.dtype)
    o = torch.empty(T, N, K, dtype=x.dtype)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("nk,nkj->nj", r[t], S + u[:, :, None] * kv)
        S = decay[t][:, :, None] * S + kv
    return _head_finish(o, w["norm"], gate, w["o"], eps)


def general_delta_mixer(x, w, m, eps):
    """Generalized delta rule: the state decays per key channel, loses a share of what it holds along the unit key,
    and gains the new key/value pair; the output reads the NEW state."""
    T = x.shape[0]
    N, K = m["heads"], m["dim"]
    r = (x @ w["r"].t()).view(T, N, K)
    k = (x @ w["k"].t()).view(T, N, K)
    v = (x @ w["v"].t()).view(T, N, K)
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(x @ w["w1"].t()) @ w["w2"].t() + w["w0"])).view(T, N, K)
    a = torch.sigmoid(x @ w["a"].t() + w["a.b"]).view(T, N, K)
    unit = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    gate = torch.sigmoid(x @ w["g"].t())
    S = torch.zeros(N, K, K, dtype=x.dtype)
    o = torch.empty(T, N, K, dtype=x.dtype)
    for t in range(T):
        held = torch.einsum("nk,nkj->nj", unit[t], S)                # what the old state holds along the unit key
        S = decay[t][:, :, None] * S - (a[t] * unit[t])[:, :, None] * held[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("nk,nkj->nj", r[t], S)
    return _head_finish(o, w["norm"], gate, w["o"], eps)


class PlainZatupel:
    def __init__(self, model_dir, dtype=torch.float64):
        with open(os.path.join(model_dir, "config.json")) as f:
            cfg = json.load(f)
        self._setup(cfg, read_safetensors(os.path.join(model_dir, "model.safetensors")), dtype)

    @classmethod
    def from_tensors(cls, cfg, tensors, dtype=torch.float64):
        """tensors: {file tensor name: numpy array or torch tensor}."""
        self = cls.__new__(cls)
        self._setup(dict(cfg), tensors, dtype)
        return self

    def _setup(self, cfg, raw, dtype):
        self.cfg, self.dtype = cfg, dtype
        self.w = {k: (v if isinstance(v, torch.Tensor) else torch.from_numpy(v)).to(dtype) for k, v in raw.items()}
        self.eps = cfg["norm"]["eps"]

    def _mixer_tensors(self, i):
        p = f"l{i}.mix."
        return {k[len(p):]: v for k, v in self.w.items() if k.startswith(p)}

    def residuals(self, ids):
        """The residual stream after every layer, [layers, T, W], and after the last one."""
        ids = torch.as_tensor(ids, dtype=torch.long)
        positions = torch.arange(ids.numel())
        x = self.w["embed"][ids] * self.cfg["embedding"]["scale"]
        v_first, after = None, []
        for i, layer in enumerate(self.cfg["layers"]):
            h = rms_norm(x, self.w[f"l{i}.norm1"], self.eps)
            mw, m = self._mixer_tensors(i), layer["mixer"]
            if layer["type"] == "attention":
                mixes = bool(m.get("v_mix"))
                y, v = attention_mixer(h, positions, mw, m, v_first if mixes else None)
                if mixes and v_first is None:
                    v_first = v
            elif layer["type"] == "wkv":
                y = wkv_mixer(h, mw, m, self.eps)
            elif layer["type"] == "general_delta":
                y = general_delta_mixer(h, mw, m, self.eps)
            else:
                raise ValueError(layer["type"])
            if layer.get("mlp") is not None:
                h2 = rms_norm(x, self.w[f"l{i}.norm2"], self.eps)
                y = y + gated_gelu(h2, self.w[f"l{i}.mlp.gate"], self.w[f"l{i}.mlp.up"], self.w[f"l{i}.mlp.down"])
            x = x + y
            after.append(x)
        return torch.stack(after), x

    def logits(self, ids):
        _, x = self.residuals(ids)
        return rms_norm(x, self.w["final.norm"], self.eps) @ self.w["head"].t()

    def generate_greedy(self, prompt, n_new):
        ids, out = list(prompt), []
        for _ in range(n_new):
            t = int(torch.argmax(self.logits(ids)[-1]))
            out.append(t)
            ids.append(t)
        return out
