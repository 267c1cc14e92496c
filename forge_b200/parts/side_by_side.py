"""Several mixers side by side: all read the same input and add their outputs into the residual stream, each times a
weight of its own (the inner mixers take it as ``out_scale``).  Each inner mixer keeps what it keeps (pages of keys and
values, a row of state, nothing); the layer's cache is the list of theirs.  ``prefixes``: what each inner mixer's tensor
names start with."""
from ..config.base import ConfigError
from .base import CompositeCacheSpec, Part, build_part, register_part


class SideBySideMixers(Part):
    graph_safe = True       # the inner mixers answer for themselves

    def __init__(self, rt, mixers):
        """mixers: list of PartSpec (category "mixer")."""
        if not mixers:
            raise ConfigError("side-by-side mixers: none given")
        self.rt = rt
        self.mixers = [build_part("mixer", spec, rt) for spec in mixers]

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

    def cache_spec(self):
        return CompositeCacheSpec(tuple(m.cache_spec() for m in self.mixers))

    def forward(self, x, batch, cache, residual):
        for m, c in zip(self.mixers, cache.parts):
            m.forward(x, batch, c, residual)


register_part("mixer", "side_by_side", SideBySideMixers, replace=True)
