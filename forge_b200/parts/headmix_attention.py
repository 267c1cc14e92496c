"""Grouped-query attention over a sliding window that also keeps the first tokens of the sequence, whose heads
exchange their weights after the softmax; optionally with values blended with an earlier layer's and a gate per head.

  [q | k | v | g] = x . [Wq; Wk; Wv; Wg]^T                       (one matrix product; g only with ``head_gate``)
  q, k <- position(q, k);   v <- (1 - lam) v + lam v_first         (``value_mix`` "blend"; "source" leaves v_first)
  cache <- k, v
  p_h(i, .) = softmax over the visible j of scale * q_h(i) . k_kv(h)(j),   visible: j <= i and (i - j < window or j < keep_first)
  w_h = sum_g mix[h, g] p_g                                         (``head_mix``)
  o_h(i) = sigmoid(g_h(i)) * sum_j w_h(i, j) v_kv(h)(j);   residual += o . Wo^T

Query/key heads and value heads may differ in size.  Every option is a constructor parameter, so another design may
take the window with kept first tokens, the exchange between heads, the value blend or the head gate alone.
"""
import torch

from .. import kernels
from ..config.base import ConfigError
from ..weights.loader import TensorSpec
from .base import KVCacheSpec, Part, build_part, register_part
from .linear import Linear

DEFAULT_NAMES = {"q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o", "head_mix": "mix.talk", "gate": "mix.g",
                 "value_mix": "mix.vmix"}


class HeadMixAttention(Part):
    graph_safe = True       # positions, tables, slots and request boundaries are read from the batch's device tensors

    def sub_parts(self):
        return [self.position]

    def __init__(self, rt, hidden_size, num_heads, num_kv_heads, head_dim, position, v_head_dim=None, scale=None, window=None,
                 keep_first=0, head_mix=True, head_gate=True, value_mix=None, value_mix_key="first_values", names=None):
        """``value_mix``: None; "source" (this layer's values, as projected, are left for later layers of the step under
        ``value_mix_key``); "blend" (this layer's values are blended with those)."""
        if num_heads % num_kv_heads:
            raise ConfigError(f"{num_heads} query heads cannot share {num_kv_heads} key/value heads")
        if value_mix not in (None, "source", "blend"):
            raise ConfigError(f"value_mix must be None, 'source' or 'blend', got {value_mix!r}")
        self.rt, self.hidden_size = rt, hidden_size
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.v_head_dim = head_dim if v_head_dim is None else v_head_dim
        self.scale = head_dim ** -0.5 if scale is None else float(scale)
        self.window, self.keep_first = window, int(keep_first or 0)
        self.head_mix, self.head_gate, self.value_mix, self.value_mix_key = bool(head_mix), bool(head_gate), value_mix, value_mix_key
        self.names = {**DEFAULT_NAMES, **(names or {})}
        self.position = build_part("position", position, rt)
        if not hasattr(self.position, "inv_freq"):
            raise ConfigError("this attention rotates inside its own prepare step and needs a position part with 'inv_freq'")
        self.proj = self.o = self.mix = self.lam = None

    def tensor_specs(self):
        n, W = self.names, self.hidden_size
        H, G, D, E = self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        specs = {n["q"]: TensorSpec((H * D, W)), n["k"]: TensorSpec((G * D, W)), n["v"]: TensorSpec((G * E, W)),
                 n["o"]: TensorSpec((W, H * E))}
        if self.head_mix:
            specs[n["head_mix"]] = TensorSpec((H, H), role="head_mix")
        if self.head_gate:
            specs[n["gate"]] = TensorSpec((H, W))
        # the blend's weight: the source layer's file may carry one that nothing reads
        specs[n["value_mix"]] = TensorSpec((), required=self.value_mix is not None, role="fraction")
        return specs

    def bind(self, tensors):
        n = self.names
        rows = [tensors[n[k]] for k in "qkv"] + ([tensors[n["gate"]]] if self.head_gate else [])
        self.proj = Linear(self._matrix(torch.cat(rows, dim=0)), None, self.rt)
        self.o = Linear(self._matrix(tensors[n["o"]]), None, self.rt)
        self.mix = self._vector_f32(tensors[n["head_mix"]]) if self.head_mix else None
        self.lam = self._vector_f32(tensors[n["value_mix"]]).reshape(1) if self.value_mix == "blend" else None

    def cache_spec(self):
        return KVCacheSpec(self.num_kv_heads, self.head_dim, self.window, v_head_dim=self.v_head_dim,
                           keep_first=self.keep_first if self.window else 0)

    def forward(self, x, batch, cache, residual):
        """x [T,W] normed input; cache: the layer's key/value pages; adds the output projection into residual."""
        H, G, D, E = self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        g = batch.groups[cache.group]
        proj = self.proj.forward(x)                                          # fp32 [T, (H+G)*D + G*E (+ H)]
        v_first = v_keep = None
        if self.value_mix == "blend":
            v_first = batch.shared.get(self.value_mix_key)
            if v_first is None:
                raise RuntimeError(f"no earlier layer of this step left {self.value_mix_key!r}")
        elif self.value_mix == "source":
            v_keep = batch.shared[self.value_mix_key] = kernels.new_tensor((x.shape[0], G * E), torch.float32, x.device,
                                                                           whole_step=True)
        q, gate = kernels.headmix_prepare(proj, batch.positions, g.slot_mapping if cache.writable else None, self.position.inv_freq,
                                          cache.kv if cache.writable else None, H, G, D, E, cache.page_size, self.rt.dtype,
                                          has_gate=self.head_gate, v_first=v_first, lam=self.lam if v_first is not None else None,
                                          v_keep=v_keep)
        o = kernels.headmix_attention(q, cache.kv, g, batch, H, G, D, E, cache.page_size, self.scale, window=self.window or 0,
                                      keep_first=self.keep_first, mix=self.mix, gate=gate)
        self.o.forward(o, accumulate_into=residual)


register_part("mixer", "headmix_attention", HeadMixAttention, replace=True)
