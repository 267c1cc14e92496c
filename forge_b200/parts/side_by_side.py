"""Several mixers side by side: all read the same input and add their outputs into the residual stream, each times a
weight of its own (the inner mixers take it as ``out_scale``).  Each inner mixer keeps what it keeps (pages of keys and
values, a row of state, nothing); the layer's cache is the list of theirs.

Inner mixers that offer it (``proj`` and ``o``, the products at their two ends, and ``mix(proj, col, batch, cache, out)``,
everything between) share ONE input product, [W_1; W_2; ...] x, and ONE output product, [O_1 | O_2 | ...] [y_1; y_2; ...], which
adds all their outputs into the stream at once; others run one after the other."""
import torch

from .. import kernels
from ..config.base import ConfigError
from .base import CompositeCacheSpec, Part, build_part, register_part
from .linear import Linear


class SideBySideMixers(Part):
    graph_safe = True       # the inner mixers answer for themselves

    def __init__(self, rt, mixers):
        """mixers: list of PartSpec (category "mixer")."""
        if not mixers:
            raise ConfigError("side-by-side mixers: none given")
        self.rt = rt
        self.mixers = [build_part("mixer", spec, rt) for spec in mixers]
        self.proj = self.o = None                    # the shared products, if the inner mixers allow them

    def sub_parts(self):
        return list(self.mixers)

    def tensor_specs(self):
        specs = {}
        for m in self.mixers:
            for name, s in m.tensor_specs().items():
                if name in specs:
                    raise ConfigError(f"side-by-side mixers: two of them name a tensor {name!r}")
                specs[name] = s
        return specs

    def bind(self, tensors):
        for m in self.mixers:
            m.bind({name: tensors[name] for name in m.tensor_specs() if name in tensors})
        ms = self.mixers
        fusable = len(ms) > 1 and all(hasattr(m, "mix") and isinstance(getattr(m, "proj", None), Linear)
                                      and isinstance(getattr(m, "o", None), Linear) for m in ms)
        # (an odd number of output columns, in all or in front of a mixer, would put its rows of the shared buffer off the
        # alignment of paired stores)
        if not fusable or any(m.out_width() % 2 for m in ms):
            return
        dev = ms[0].proj.weight.device

        def bias_of(lin, n):
            return lin.bias if lin.bias is not None else torch.zeros(n, dtype=torch.float32, device=dev)
        b_in = torch.cat([bias_of(m.proj, m.in_width()) for m in ms]) if any(m.proj.bias is not None for m in ms) else None
        b_out = sum(m.o.bias for m in ms if m.o.bias is not None) if any(m.o.bias is not None for m in ms) else None
        self.proj = Linear(torch.cat([m.proj.weight for m in ms], dim=0).contiguous(), b_in, self.rt)
        self.o = Linear(torch.cat([m.o.weight for m in ms], dim=1).contiguous(), b_out, self.rt)
        for m in ms:                                  # the inner mixers' own copies are not needed any more
            m.proj = m.o = None

    def cache_spec(self):
        return CompositeCacheSpec(tuple(m.cache_spec() for m in self.mixers))

    def forward(self, x, batch, cache, residual):
        if self.proj is None:
            for m, c in zip(self.mixers, cache.parts):
                m.forward(x, batch, c, residual)
            return
        p = self.proj.forward(x)                      # fp32 [T, all inner projections side by side]
        y = kernels.new_tensor((x.shape[0], self.o.in_features), self.rt.dtype, x.device)
        col = ycol = 0
        for m, c in zip(self.mixers, cache.parts):
            m.mix(p, col, batch, c, out=(y, ycol))
            col, ycol = col + m.in_width(), ycol + m.out_width()
        self.o.forward(y, accumulate_into=residual)


register_part("mixer", "side_by_side", SideBySideMixers, replace=True)
