"""Small Zatupel configurations for the tests, and model folders with random weights made from them.

The three differ in every size, in the order and number of the layers and in every constant; among them they have
what a single model can hide: value heads as large as key heads and not; as many key/value heads as query heads, fewer,
one; a rotation over the whole head and over a part; no kept first tokens; a window longer than any test sequence; a layer
without a feed-forward; an attention layer that blends no values beside ones that do; a state mixer as first layer;
state heads whose channels do not add up to the model's width; several layers of each kind; head sizes that are no powers
of two.
"""
import copy
import math

import torch

from forge_b200.config import config_from_dict
from forge_b200.weights import write_random_model


def _att(heads, kv, dim, vdim, size, keep, rot, base, v_mix, scale=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "v_mix": v_mix,
                                           "mask": {"size": size, "keep_first": keep}, "rot": {"dims": rot, "base": base},
                                           "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}}


def _state(kind, heads, dim, rank):
    return {"type": kind, "mixer": {"heads": heads, "dim": dim, "rank": rank}}


def _with_mlp(layer, ff):
    return dict(layer, mlp=None if ff is None else {"kind": "dense", "ff": ff})


ZAT = {
    "P": {"architecture": "Zatupel", "vocab": 211, "width": 80, "embedding": {"scale": 1.7}, "norm": {"eps": 1e-5},
          "layers": [_with_mlp(_state("wkv", 5, 16, 8), 96),
                     _with_mlp(_att(6, 3, 24, 24, 20, 3, 16, 5000.0, True, 0.3), 112),
                     _with_mlp(_state("general_delta", 3, 24, 12), None),
                     _with_mlp(_att(6, 3, 24, 24, 11, 0, 24, 800.0, True), 72),
                     _with_mlp(_att(4, 4, 16, 40, 500, 2, 8, 100.0, False), 64),
                     _with_mlp(_att(6, 3, 24, 24, 33, 9, 12, 1e6, True), 88)]},
    "Q": {"architecture": "Zatupel", "vocab": 130, "width": 48, "embedding": {"scale": 0.25}, "norm": {"eps": 1e-3},
          "layers": [_with_mlp(_att(3, 1, 16, 8, 9, 1, 16, 30.0, False, 0.4), 40),
                     _with_mlp(_state("general_delta", 2, 32, 4), 56),
                     _with_mlp(_state("general_delta", 4, 8, 16), 56),
                     _with_mlp(_state("wkv", 1, 40, 24), None),
                     _with_mlp(_state("wkv", 3, 16, 8), 40)]},
    # widths at which the bfloat16 path takes the tensor-core products (every reduction a multiple of 8)
    "R": {"architecture": "Zatupel", "vocab": 520, "width": 256, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
          "layers": [_with_mlp(_att(8, 2, 64, 32, 70, 5, 32, 10000.0, True), 384),
                     _with_mlp(_state("wkv", 4, 64, 32), 384),
                     _with_mlp(_att(8, 2, 64, 32, 40, 0, 64, 250000.0, True), 384),
                     _with_mlp(_state("general_delta", 2, 64, 16), 256)]},
}
SEEDS = {"P": 11, "Q": 12, "R": 13}
# weights large enough that attention is far from uniform, decays and removal rates spread over (0, 1) and every norm
# weight, bias, bonus and blend matters
STDS = {"P": dict(std=0.14, embed_std=0.6, norm_std=0.2, bias_std=0.7), "Q": dict(std=0.2, embed_std=0.8, norm_std=0.2, bias_std=0.7),
        "R": dict(std=0.08, embed_std=0.6, norm_std=0.2, bias_std=0.7)}
LENGTHS = {"P": [70, 129, 33, 150, 64, 97], "Q": [90, 47, 16, 140, 81], "R": [160, 20, 131, 45]}


def zat_config(name):
    return config_from_dict(copy.deepcopy(ZAT[name]))


def make_zat_dir(tmp_path_factory, name):
    d = str(tmp_path_factory.mktemp(f"zat{name}"))
    write_random_model(zat_config(name), d, seed=SEEDS[name], **STDS[name])
    return d


def rand(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale
