"""Small Tidenex configurations for the tests, and model folders with random weights made from them.

The three differ in every size, in the order and number of the layers, in the span that repeats and in every constant;
among them they have what a single model can hide: value heads as wide as a head's two maps together and not; as many
key/value heads as query heads, fewer, one; a rotation over a part of a map, over all of it and none; a difference weight
of zero; a temperature that changes at every position and one that never changes within a test; state heads with more key
than value channels and the reverse, with channel counts that are no multiple of four; mixer weights above and below one;
a layer without a feed-forward; no repeated span, a span that starts at the first layer, a span of one layer run four times.
"""
import copy

from forge_b200.config import config_from_dict
from forge_b200.weights import write_random_model


def _att(heads, kv, dim, vdim, rot, base, scale, diff):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "rot": {"dims": rot, "base": base},
                                           "scale": scale, "diff": diff}}


def _par(lh, lg, ld, lv, lscale, temp, rh, rd, rv, ls, rs):
    left = {"heads": lh, "kv_heads": lg, "dim": ld, "vdim": lv, "scale": lscale}
    if temp is not None:
        left["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return {"type": "parallel", "mixer": {"left": left, "right": {"heads": rh, "dim": rd, "vdim": rv}, "left_scale": ls, "right_scale": rs}}


def _with_mlp(layer, ff):
    return dict(layer, mlp=None if ff is None else {"kind": "dense", "ff": ff})


TID = {
    "X": {"architecture": "Tidenex", "vocab": 211, "width": 80, "norm": {"eps": 1e-4}, "loop": {"start": 1, "stop": 3, "times": 3},
          "layers": [_with_mlp(_par(4, 1, 24, 8, 0.2, (0.5, 7), 5, 12, 20, 1.3, 0.6), 96),
                     _with_mlp(_att(6, 3, 16, 24, 8, 300.0, 0.3, 0.35), 112),
                     _with_mlp(_att(3, 3, 8, 16, 8, 5000.0, 0.4, 0.8), None),
                     _with_mlp(_par(2, 2, 16, 16, 0.25, (0.2, 1), 3, 10, 6, 0.7, 1.5), 72)]},
    "Y": {"architecture": "Tidenex", "vocab": 130, "width": 48, "norm": {"eps": 1e-2},
          "layers": [_with_mlp(_att(2, 1, 24, 8, 0, 10.0, 0.2, 0.0), 40),
                     _with_mlp(_par(3, 3, 8, 40, 0.5, None, 1, 40, 24, 1.0, 1.0), None),
                     _with_mlp(_att(4, 2, 12, 12, 12, 1e6, 0.3, 0.5), 56)]},
    # widths at which the bfloat16 path takes the tensor-core products (every reduction a multiple of 8)
    "Z": {"architecture": "Tidenex", "vocab": 520, "width": 256, "norm": {"eps": 1e-6}, "loop": {"start": 0, "stop": 1, "times": 4},
          "layers": [_with_mlp(_par(4, 2, 32, 64, 0.18, (0.35, 50), 4, 64, 32, 0.9, 1.2), 384),
                     _with_mlp(_att(8, 2, 32, 32, 16, 10000.0, 0.18, 0.4), 384)]},
}
SEEDS = {"X": 21, "Y": 22, "Z": 23}
STDS = {"X": dict(std=0.14, embed_std=0.6, norm_std=0.2, bias_std=0.4), "Y": dict(std=0.2, embed_std=0.8, norm_std=0.2, bias_std=0.4),
        "Z": dict(std=0.08, embed_std=0.6, norm_std=0.2, bias_std=0.4)}
LENGTHS = {"X": [70, 129, 33, 150, 64, 97], "Y": [90, 47, 16, 140, 81], "Z": [160, 20, 131, 45]}


def tid_config(name):
    return config_from_dict(copy.deepcopy(TID[name]))


def make_tid_dir(tmp_path_factory, name):
    d = str(tmp_path_factory.mktemp(f"tid{name}"))
    write_random_model(tid_config(name), d, seed=SEEDS[name], **STDS[name])
    return d
