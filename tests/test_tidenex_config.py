"""Tidenex on the CPU: configuration, plan, tensor names, refusals, cache needs, and the plain implementation against itself."""
import copy
import math

import pytest
import torch

from forge_b200.cache.storage import bytes_per_page, plan_groups
from forge_b200.config import ConfigError, config_from_dict
from forge_b200.engine.model import Model
from forge_b200.parts import CompositeCacheSpec, KVCacheSpec, Runtime, StateSpec
from plain import tidenex as PT
from tidenex_models import TID, tid_config
from zatupel_models import rand


def _model(name):
    return Model(tid_config(name).plan(), Runtime(torch.device("cpu"), torch.bfloat16))


def test_schedule_and_where_the_embedding_comes_in_again():
    p = tid_config("X").plan()
    assert p.schedule == [0, 1, 2, 1, 2, 1, 2, 3] and p.add_embedding_before == (3, 5)
    p = tid_config("Y").plan()
    assert p.schedule == [0, 1, 2] and p.add_embedding_before == ()
    p = tid_config("Z").plan()
    assert p.schedule == [0, 0, 0, 0, 1] and p.add_embedding_before == (1, 2, 3)
    assert [i for i, again in PT.schedule_of(TID["X"])] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [k for k, (i, again) in enumerate(PT.schedule_of(TID["Z"])) if again] == [1, 2, 3]


def test_tensor_names_and_shapes():
    specs = _model("X").tensor_specs()
    for name, shape in {"embed": (211, 80), "final.norm": (80,), "final.norm.b": (80,), "l0.norm1.b": (80,), "l0.mix.left.q": (96, 80),
                        "l0.mix.left.k.b": (24,), "l0.mix.left.v": (8, 80), "l0.mix.left.q.norm": (96,), "l0.mix.left.r2": (4,),
                        "l0.mix.left.o": (80, 32), "l0.mix.left.o.b": (80,), "l0.mix.right.f": (60, 80), "l0.mix.right.lower": (60,),
                        "l0.mix.right.v": (100, 80), "l0.mix.right.norm": (20,), "l0.mix.right.o": (80, 100),
                        "l1.mix.q": (192, 80), "l1.mix.k": (96, 80), "l1.mix.v": (72, 80), "l1.mix.lk2": (16,), "l1.mix.o": (80, 144),
                        "l1.mlp.up": (112, 80), "l1.mlp.down": (80, 112), "l2.norm1": (80,)}.items():
        assert tuple(specs[name].shape) == shape, name
    assert "l2.norm2" not in specs and "l2.mlp.up" not in specs          # a layer without a feed-forward has one norm
    assert not specs["head"].required                                      # the head is the embedding table


def test_every_run_of_a_repeated_layer_keeps_a_cache_of_its_own():
    m = _model("X")
    specs = m.cache_specs()
    assert len(specs) == 8
    assert isinstance(specs[0], CompositeCacheSpec) and isinstance(specs[0].parts[0], KVCacheSpec) and isinstance(specs[0].parts[1], StateSpec)
    assert specs[0].parts[1].shape == (5 * 12 * 20,)
    assert specs[1] == KVCacheSpec(3, 32, None, v_head_dim=24) and specs[3] == specs[1] and specs[2] == KVCacheSpec(3, 16, None, v_head_dim=16)
    groups, _ = plan_groups(specs, m.cache_from())
    assert len(groups) == 4
    per_page = bytes_per_page(specs, m.cache_from(), 8, torch.bfloat16)
    assert per_page["kv3x32v24_full"] == 3 * 3 * 8 * (32 + 24) * 2          # three runs of layer 1


@pytest.mark.parametrize("change, message", [
    (lambda d: d["layers"][1].update(type="conv"), "type"),
    (lambda d: d["layers"][1]["mixer"].update(kv_heads=4), "kv_heads"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda d: d["layers"][1]["mixer"].update(diff=1.0), "diff"),
    (lambda d: d["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda d: d["layers"][0]["mixer"].update(left_scale="big"), "left_scale"),
    (lambda d: d["layers"][0]["mixer"]["left"]["q_temp"].update(every=0), "q_temp"),
    (lambda d: d["layers"][0]["mlp"].update(kind="moe"), "mlp.kind"),
    (lambda d: d["loop"].update(stop=9), "loop"),
    (lambda d: d["loop"].update(times=0), "loop"),
    (lambda d: d.pop("norm"), "norm"),
])
def test_refusals(change, message):
    d = copy.deepcopy(TID["X"])
    change(d)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(d)


def test_what_config_does_not_mention_does_not_exist():
    d = copy.deepcopy(TID["X"])
    d["layers"][1]["mixer"].pop("rot")
    d["layers"][0]["mixer"].pop("right_scale")
    d["layers"][0]["mixer"]["left"].pop("q_temp")
    p = config_from_dict(d).plan()
    assert p.layers[1].mixer.params["position"].params["rotary_dims"] == 0
    inner = p.layers[0].mixer.params["mixers"]
    assert inner[1].params["out_scale"] == 1.0 and inner[0].params["out_scale"] == 1.3 and inner[0].params["temp_every"] == 0.0


def test_to_dict_round_trip():
    for name in TID:
        c = tid_config(name)
        assert config_from_dict(c.to_dict()) == c


# ------------------------------------------------------------------------------------- the plain implementation against itself

def test_plain_rotation_turns_pairs_half_apart_and_leaves_the_rest():
    x = rand(5, 2, 12, seed=1).double()
    pos = torch.tensor([0, 1, 2, 50, 1000])
    y = PT.rotate_halves(x, pos, 100.0, 8)
    assert torch.equal(y[..., 8:], x[..., 8:]) and torch.equal(y[0], x[0])
    for i in range(4):
        a = pos.double() * 100.0 ** (-2.0 * i / 8)
        u, v = x[:, :, i], x[:, :, i + 4]
        assert torch.allclose(y[:, :, i], u * torch.cos(a)[:, None] - v * torch.sin(a)[:, None], atol=1e-12)
        assert torch.allclose(y[:, :, i + 4], v * torch.cos(a)[:, None] + u * torch.sin(a)[:, None], atol=1e-12)
    assert torch.allclose((y ** 2).sum(-1), (x ** 2).sum(-1), atol=1e-9)


def test_plain_mixers_do_not_look_ahead():
    W, T = 32, 40
    h = rand(T, W, seed=2).double()
    h2 = h.clone()
    h2[25:] = rand(T - 25, W, seed=3).double()
    m_att = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "rot": {"dims": 4, "base": 50.0}, "scale": 0.3, "diff": 0.3}
    w = {"q": rand(64, W, seed=4), "k": rand(32, W, seed=5), "v": rand(24, W, seed=6), "o": rand(W, 48, seed=7),
         "lq1": rand(8, seed=8, scale=0.3), "lk1": rand(8, seed=9, scale=0.3), "lq2": rand(8, seed=10, scale=0.3), "lk2": rand(8, seed=11, scale=0.3)}
    w = {k: v.double() * 0.3 for k, v in w.items()}
    assert torch.allclose(PT.differential_attention(h, w, m_att, 1e-5)[:25], PT.differential_attention(h2, w, m_att, 1e-5)[:25], atol=1e-10)
    m_r = {"heads": 2, "dim": 6, "vdim": 10}
    wr = {"q": rand(12, W, seed=12), "f": rand(12, W, seed=13), "f.b": rand(12, seed=14), "lower": torch.rand(12), "v": rand(20, W, seed=15),
          "norm": torch.ones(10), "o": rand(W, 20, seed=16)}
    wr = {k: v.double() for k, v in wr.items()}
    a, _ = PT.gated_linear_recurrence(h, wr, m_r, 1e-5)
    b, _ = PT.gated_linear_recurrence(h2, wr, m_r, 1e-5)
    assert torch.allclose(a[:25], b[:25], atol=1e-10)
    # carried over two calls the state gives what one call gives
    first, S = PT.gated_linear_recurrence(h[:17], wr, m_r, 1e-5)
    second, _ = PT.gated_linear_recurrence(h[17:], wr, m_r, 1e-5, state=S)
    assert torch.allclose(torch.cat([first, second]), a, atol=1e-10)


def test_plain_recurrence_with_a_gate_of_one_keeps_and_of_the_bound_writes():
    """A lower bound of 1 freezes the (empty) state: the output is zero.  A huge negative gate input leaves f at its bound."""
    W, T = 8, 5
    h = rand(T, W, seed=20).double()
    m = {"heads": 1, "dim": 4, "vdim": 4}
    w = {"q": rand(4, W, seed=21).double(), "f": torch.zeros(4, W).double(), "f.b": torch.full((4,), -50.0).double(),
         "lower": torch.ones(4).double(), "v": rand(4, W, seed=22).double(), "norm": torch.ones(4).double(), "o": torch.eye(W, 4).double()}
    out, S = PT.gated_linear_recurrence(h, w, m, 1e-5)
    assert float(out.abs().max()) == 0.0 and float(S.abs().max()) == 0.0
    w["lower"] = torch.full((4,), 0.25).double()
    _, S = PT.gated_linear_recurrence(h[:1], w, m, 1e-5)
    v0 = h[0] @ w["v"].t()
    assert torch.allclose(S[0], 0.75 * v0[None, :].expand(4, 4), atol=1e-12)


def test_plain_distance_term_and_temperature():
    """With zero queries the weights are (1 + r2 d)^(-r1) over the distance d; the temperature multiplies q."""
    W, T = 8, 30
    h = rand(T, W, seed=30).double()
    m = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 1.0, "q_temp": {"coef": 0.5, "every": 4}}
    w = {"q": torch.zeros(4, W), "q.b": torch.zeros(4), "k": rand(4, W, seed=31), "k.b": torch.zeros(4), "v": rand(4, W, seed=32),
         "v.b": torch.zeros(4), "q.norm": torch.ones(4), "k.norm": torch.ones(4), "r1": torch.tensor([1.5]), "r2": torch.tensor([0.7]),
         "o": torch.eye(W, 4), "o.b": torch.zeros(W)}
    w = {k: v.double() for k, v in w.items()}
    out = PT.biased_attention(h, w, m, 1e-6)
    v = h @ w["v"].t()
    i = 17
    wt = torch.tensor([(1 + 0.7 * (i - j)) ** -1.5 for j in range(i + 1)]).double()
    assert torch.allclose(out[i, :4], (wt[:, None] * v[:i + 1]).sum(0) / wt.sum(), atol=1e-10)
    assert math.isclose(1.0 + 0.5 * math.log(math.floor((11 + 1) / 4) + 1), 1.0 + 0.5 * math.log(4.0))
