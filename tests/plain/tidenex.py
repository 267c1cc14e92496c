"""Whole-sequence Tidenex decoder, written from the design's equations: one request, all of its tokens, every
time; no cache, no state carried over calls, no batching, no fusing.  float64 on the CPU.  One function per mechanism.

Notation: T tokens, W model width, H query heads, G key/value heads, D query/key size of a head (of one map), E value
size of a head, N heads of the recurrent mixer with K key and V value channels.
"""
import json
import math
import os

import torch

from .safetensors_reader import read_safetensors


def layer_norm(x, weight, bias, eps):
    """(x - mean) / sqrt(mean of squared deviations + eps) * weight + bias over the last dimension."""
    mu = x.mean(dim=-1, keepdim=True)
    var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * weight + bias


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def dense_ff(x, w_up, w_down):
    return gelu_erf(x @ w_up.t()) @ w_down.t()


def rotate_halves(x, positions, base, dims):
    """Rotary encoding of x[T, heads, D] on its first ``dims`` channels, channel i paired with i + dims/2;
    angle = position * base^(-2i/dims).  The other channels pass unchanged."""
    out = x.clone()
    if dims == 0:
        return out
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = torch.pow(torch.tensor(float(base), dtype=x.dtype), -2.0 * i / dims)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def causal_softmax(scores):
    """scores [H, T, T]: softmax over the keys j <= i."""
    T = scores.shape[-1]
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    return torch.softmax(scores.masked_fill(~mask, float("-inf")), dim=-1)


def differential_attention(h, w, m, eps):
    """h [T, W]; w: {"q","k","v","o","lq1","lk1","lq2","lk2"}; m: the mixer's numbers.  Two softmax maps per head over the
    same values, o = a1 - lambda a2, divided by its root mean square over the head's values, times (1 - diff)."""
    T = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ w["q"].t()).view(T, H * 2, D)
    k = (h @ w["k"].t()).view(T, G * 2, D)
    v = (h @ w["v"].t()).view(T, G, E)
    rot = m.get("rot") or {"base": 1.0, "dims": 0}          # a mixer without the key has no rotation
    q = rotate_halves(q, pos, rot["base"], rot["dims"]).view(T, H, 2, D)
    k = rotate_halves(k, pos, rot["base"], rot["dims"]).view(T, G, 2, D)
    lam = math.exp(float((w["lq1"] * w["lk1"]).sum())) - math.exp(float((w["lq2"] * w["lk2"]).sum())) + m["diff"]
    rep = H // G
    out = torch.zeros(T, H, E, dtype=h.dtype)
    for head in range(H):
        g = head // rep
        a = []
        for mp in range(2):
            s = (q[:, head, mp] @ k[:, g, mp].t()) * m["scale"]
            a.append(causal_softmax(s[None])[0] @ v[:, g])
        o = a[0] - lam * a[1]
        out[:, head] = rms_unit(o, eps) * (1.0 - m["diff"])
    return out.reshape(T, H * E) @ w["o"].t()


def biased_attention(h, w, m, eps):
    """Softmax attention without rotation: biases in every projection, RMS norm over the whole of q and of k with
    weights, a query temperature that grows with the position, a distance bias per head taken off the scores."""
    T = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_unit(h @ w["q"].t() + w["q.b"], eps) * w["q.norm"]
    k = rms_unit(h @ w["k"].t() + w["k.b"], eps) * w["k.norm"]
    v = (h @ w["v"].t() + w["v.b"]).view(T, G, E)
    p = torch.arange(T, dtype=h.dtype)
    temp = torch.ones(T, dtype=h.dtype)
    if m.get("q_temp"):                      # a mixer without the key has no temperature
        temp = 1.0 + m["q_temp"]["coef"] * torch.log(torch.floor((p + 1) / m["q_temp"]["every"]) + 1.0)
    q = (q * temp[:, None]).view(T, H, D)
    k = k.view(T, G, D)
    dist = (p[:, None] - p[None, :]).clamp(min=0)
    rep = H // G
    out = torch.zeros(T, H, E, dtype=h.dtype)
    for head in range(H):
        g = head // rep
        s = (q[:, head] @ k[:, g].t()) * m["scale"] - w["r1"][head] * torch.log1p(w["r2"][head] * dist)
        out[:, head] = causal_softmax(s[None])[0] @ v[:, g]
    return out.reshape(T, H * E) @ w["o"].t() + w["o.b"]


def gated_linear_recurrence(h, w, m, eps, state=None):
    """HGRN2: S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t per head, f bounded below; each head's output RMS
    normed with a weight shared by the heads.  Returns (output [T, W], final state [N, K, V])."""
    T = h.shape[0]
    N, K, V = m["heads"], m["dim"], m["vdim"]
    q = torch.nn.functional.silu(h @ w["q"].t()).view(T, N, K)
    v = (h @ w["v"].t()).view(T, N, V)
    low = w["lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ w["f"].t() + w["f.b"])).view(T, N, K)
    S = torch.zeros(N, K, V, dtype=h.dtype) if state is None else state.clone()
    out = torch.zeros(T, N, V, dtype=h.dtype)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("nkv,nk->nv", S, q[t])
    out = rms_unit(out, eps) * w["norm"]
    return out.reshape(T, N * V) @ w["o"].t(), S


def parallel_mixer(h, w, m, eps):
    left = biased_attention(h, {k[5:]: v for k, v in w.items() if k.startswith("left.")}, m["left"], eps)
    right, _ = gated_linear_recurrence(h, {k[6:]: v for k, v in w.items() if k.startswith("right.")}, m["right"], eps)
    return m.get("left_scale", 1.0) * left + m.get("right_scale", 1.0) * right


MIXERS = {"attention": differential_attention, "parallel": parallel_mixer}


def schedule_of(config):
    """[(layer, first of a repeated pass)] in the order the layers run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    out = [(i, False) for i in range(a)]
    for p in range(times):
        out += [(i, p > 0 and i == a) for i in range(a, b)]
    return out + [(i, False) for i in range(b, n)]


class PlainTidenex:
    def __init__(self, config, tensors, dtype=torch.float64):
        self.c = config
        self.t = {k: torch.as_tensor(v).to(dtype) for k, v in tensors.items()}
        self.dtype = dtype

    @classmethod
    def from_dir(cls, path, dtype=torch.float64):
        with open(os.path.join(path, "config.json")) as f:
            config = json.load(f)
        return cls(config, read_safetensors(os.path.join(path, "model.safetensors")), dtype)

    def layer(self, i, x):
        c, t, eps = self.c["layers"][i], self.t, self.c["norm"]["eps"]
        pre = f"l{i}."
        w = {k[len(pre) + 4:]: v for k, v in t.items() if k.startswith(pre + "mix.")}
        x = x + MIXERS[c["type"]](layer_norm(x, t[pre + "norm1"], t[pre + "norm1.b"], eps), w, c["mixer"], eps)
        if c.get("mlp") is not None:
            x = x + dense_ff(layer_norm(x, t[pre + "norm2"], t[pre + "norm2.b"], eps), t[pre + "mlp.up"], t[pre + "mlp.down"])
        return x

    def forward(self, tokens, keep_layers=False):
        """logits [T, vocab] of one whole sequence (and the residual stream after every layer run)."""
        t = self.t
        x0 = t["embed"][torch.as_tensor(tokens, dtype=torch.long)]
        x, streams = x0, []
        for i, again in schedule_of(self.c):
            if again:
                x = x + x0
            x = self.layer(i, x)
            streams.append(x)
        y = layer_norm(x, t["final.norm"], t["final.norm.b"], self.c["norm"]["eps"])
        logits = y @ t["embed"].t()
        return (logits, torch.stack(streams)) if keep_layers else logits
