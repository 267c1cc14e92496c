"""The Zatupel configuration, its plan and tensor names, the pieces of the cache manager that it brought (kept first
positions of a windowed group, value heads of another size), sizes that only the file's tensors give, and the plain
implementation's mechanisms against each other.  No GPU."""
import copy
import json
import math
import os

import pytest
import torch

from forge_b200.cache import CacheManager
from forge_b200.cache.manager import GroupSpec
from forge_b200.config import ConfigError, ZatupelConfig, config_from_dict, load_config
from forge_b200.engine.model import Model
from forge_b200.parts import Runtime
from forge_b200.weights import WeightError, write_random_model
from forge_b200.weights.loader import TensorSpec, check_tensors, load_tensors
from plain import llama as PL
from plain import zatupel as PZ
from plain.safetensors_reader import read_safetensors
from zatupel_models import SEEDS, STDS, ZAT, rand, zat_config


def _model(cfg):
    return Model(cfg.plan(), Runtime(torch.device("cpu"), torch.float32))


def test_one_string_names_the_architecture():
    cfg = zat_config("P")
    assert isinstance(cfg, ZatupelConfig) and cfg.num_hidden_layers == 6 and cfg.hidden_size == 80 and cfg.vocab_size == 211
    assert config_from_dict(cfg.to_dict()) == cfg


def test_plan_reads_every_constant_from_the_configuration():
    plan = zat_config("P").plan()
    assert [l.mixer.kind for l in plan.layers] == ["wkv", "headmix_attention", "general_delta", "headmix_attention",
                                                   "headmix_attention", "headmix_attention"]
    assert [l.block for l in plan.layers] == ["parallel"] * 6 and plan.embedding.params["scale"] == 1.7
    a = plan.layers[1].mixer.params
    assert (a["num_heads"], a["num_kv_heads"], a["head_dim"], a["v_head_dim"], a["window"], a["keep_first"], a["scale"]) == (6, 3, 24, 24, 20, 3, 0.3)
    assert a["position"].params == {"head_dim": 24, "rotary_dims": 16, "theta": 5000.0}
    # the first layer that blends values is their source; a layer that does not blend stands outside
    assert [plan.layers[i].mixer.params["value_mix"] for i in (1, 3, 4, 5)] == ["source", "blend", None, "blend"]
    assert plan.layers[2].feed_forward.kind == "none" and plan.layers[2].norms["feed_forward"] is None
    assert plan.layers[0].feed_forward.params["intermediate_size"] == 96
    assert plan.final_norm.params["eps"] == 1e-5 and plan.layers[3].norms["mixer"].params["eps"] == 1e-5


def test_tensor_names_and_shapes():
    specs = _model(zat_config("Q")).tensor_specs()
    assert specs["embed"].shape == (130, 48) and specs["head"].shape == (130, 48) and specs["final.norm"].shape == (48,)
    assert specs["l0.mix.q"].shape == (48, 48) and specs["l0.mix.k"].shape == (16, 48) and specs["l0.mix.v"].shape == (8, 48)
    assert specs["l0.mix.o"].shape == (48, 24) and specs["l0.mix.talk"].shape == (3, 3) and specs["l0.mix.g"].shape == (3, 48)
    assert specs["l0.mix.vmix"].shape == () and not specs["l0.mix.vmix"].required
    assert specs["l1.mix.a.b"].shape == (64,) and specs["l1.mix.w1"].shape == (-1, 48) and specs["l1.mix.w2"].shape == (64, -1)
    assert specs["l3.mix.mu.w"].shape == (48,) and specs["l3.mix.u"].shape == (1, 40) and specs["l3.mix.o"].shape == (48, 40)
    assert "l3.norm2" not in specs and "l3.mlp.gate" not in specs and specs["l4.mlp.down"].shape == (48, 40)


@pytest.mark.parametrize("patch, needle", [
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d["layers"][0].update(type="conv"), "type"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=2), "kv_heads"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda d: d["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda d: d["layers"][1].update(mlp={"kind": "routed", "ff": 8}), "mlp.kind"),
    (lambda d: d.update(layers=[]), "layers"),
    (lambda d: d["norm"].pop("eps"), "eps"),
])
def test_bad_configurations_are_refused(patch, needle):
    d = copy.deepcopy(ZAT["Q"])
    patch(d)
    with pytest.raises(ConfigError, match=needle):
        config_from_dict(d)


def test_random_folder_loads_and_the_file_gives_the_rank(tmp_path):
    cfg = zat_config("Q")
    d = write_random_model(cfg, str(tmp_path), seed=SEEDS["Q"], **STDS["Q"])
    assert json.load(open(os.path.join(d, "config.json")))["architecture"] == "Zatupel"
    assert load_config(d) == cfg
    # the configuration that a user's file has says nothing of the rank: the tensors do
    bare = copy.deepcopy(ZAT["Q"])
    for layer in bare["layers"]:
        layer["mixer"].pop("rank", None)
    model = _model(config_from_dict(bare))
    tensors = load_tensors(d, model.tensor_specs())
    assert tensors["l1.mix.w1"].shape == (4, 48) and tensors["l2.mix.w2"].shape == (32, 16)
    model.load(tensors)
    assert model.blocks[1].mixer.w2.in_features == 4 and model.blocks[3].mixer.w1.out_features == 24
    raw = read_safetensors(os.path.join(d, "model.safetensors"))
    assert "l0.mix.vmix" not in raw and raw["l0.mix.talk"].shape == (3, 3)       # a layer that blends nothing has no weight for it


def test_a_number_without_dimensions_is_written_and_read(tmp_path):
    d = write_random_model(zat_config("P"), str(tmp_path), seed=1)
    raw = read_safetensors(os.path.join(d, "model.safetensors"))
    assert raw["l3.mix.vmix"].shape == () and 0.0 <= float(raw["l3.mix.vmix"]) <= 1.0 and "l4.mix.vmix" not in raw
    model = _model(load_config(d))
    model.load(load_tensors(d, model.tensor_specs()))
    assert model.blocks[3].mixer.lam.shape == (1,) and model.blocks[1].mixer.lam is None


def test_sizes_left_to_the_file_must_still_agree():
    specs = {"a": TensorSpec((-1, 6)), "b": TensorSpec((5, -1))}
    check_tensors("x", specs, {"a": ((3, 6), torch.float32), "b": ((5, 9), torch.float32)})
    with pytest.raises(WeightError, match="wrong shape"):
        check_tensors("x", specs, {"a": ((3, 7), torch.float32), "b": ((5, 9), torch.float32)})
    with pytest.raises(WeightError, match="wrong shape"):
        check_tensors("x", specs, {"a": ((3, 6, 1), torch.float32), "b": ((5, 9), torch.float32)})


def test_cache_needs():
    from forge_b200.cache.storage import bytes_per_page, plan_groups
    model = _model(zat_config("P"))
    specs = model.cache_specs()
    assert specs[0].shape == (5 * 16 * 16 + 80,) and specs[2].shape == (3 * 24 * 24,)
    assert (specs[1].num_kv_heads, specs[1].head_dim, specs[1].value_dim, specs[1].window, specs[1].keep_first) == (3, 24, 24, 20, 3)
    assert (specs[4].head_dim, specs[4].value_dim, specs[4].window, specs[4].keep_first) == (16, 40, 500, 2)
    groups, per_layer = plan_groups(specs, [None] * 6)
    assert len(groups) == 4 and per_layer[0] is None and len({per_layer[i] for i in (1, 3, 4, 5)}) == 4
    assert bytes_per_page(specs, [None] * 6, 8, torch.float32)[per_layer[4]] == 4 * 8 * (16 + 40) * 4


def test_kept_first_pages_are_never_given_back():
    m = CacheManager([GroupSpec("w", 12, window=10, keep_first=5), GroupSpec("plain", 12, window=10)], page_size=4, max_requests=2)
    m.admit("r")
    m.append("r", 30)
    assert m.release_out_of_window("r") == 3 + 5
    # positions 0..4 live in pages 0 and 1: they stay; pages 2..4 (positions 8..19) are behind every window
    assert m.block_table("r", "w")[:6] == [0, 1, -1, -1, -1, 5] and m.block_table("r", "plain")[:6] == [-1] * 5 + [5]
    m.check()
    m.append("r", 10)
    m.release_out_of_window("r")
    assert m.block_table("r", "w")[:2] == [0, 1] and m.block_table("r", "w")[2:7] == [-1] * 5
    m.free("r")
    m.check()
    assert m.num_free_pages() == {"w": 12, "plain": 12}


# ------------------------------------------------------------------------ the plain implementation against itself

def test_plain_attention_without_its_extras_is_ordinary_windowed_attention():
    T, H, G, D = 40, 4, 2, 8
    q, k, v = rand(T, H, D, seed=1).double(), rand(T, G, D, seed=2).double(), rand(T, G, D, seed=3).double()
    want = PL.attention(q, k, v, window=7)
    got = PZ.mixed_head_attention(q, k, v, 1.0 / math.sqrt(D), 7, 0, torch.eye(H, dtype=torch.float64))
    assert torch.allclose(got, want, atol=1e-12)
    # kept first tokens: the rows that no longer reach them through the window change, the early rows do not
    kept = PZ.mixed_head_attention(q, k, v, 1.0 / math.sqrt(D), 7, 3, torch.eye(H, dtype=torch.float64))
    assert torch.allclose(kept[:7], want[:7], atol=1e-12) and not torch.allclose(kept[7:8], want[7:8], atol=1e-3)


def test_plain_mask_edges():
    m = PZ.visible(30, 5, 2)
    assert m[20, 16] and not m[20, 15] and m[20, 1] and not m[20, 2] and m[20, 20] and not m[20, 21]
    assert m[3, 0] and m[4, 0] and m[6, 1] and m[6, 2] and not m[7, 2]


def test_plain_rotation_is_a_rotation_of_neighbours():
    x = rand(5, 2, 12, seed=4).double()
    y = PZ.rotate_neighbours(x, torch.arange(5), 100.0, 8)
    assert torch.equal(y[..., 8:], x[..., 8:]) and torch.equal(y[0], x[0])
    assert torch.allclose((y[..., 0:8:2] ** 2 + y[..., 1:8:2] ** 2), (x[..., 0:8:2] ** 2 + x[..., 1:8:2] ** 2), atol=1e-12)
    # pair 0 turns by the position itself: position 3, channels (0, 1)
    a, b = x[3, 0, 0], x[3, 0, 1]
    assert torch.allclose(y[3, 0, 0], a * math.cos(3) - b * math.sin(3)) and torch.allclose(y[3, 0, 1], b * math.cos(3) + a * math.sin(3))


def test_plain_state_mixers_do_not_look_ahead():
    cfg = ZAT["Q"]
    W = cfg["width"]
    x = rand(12, W, seed=5).double()
    for i, fn in ((3, PZ.wkv_mixer), (1, PZ.general_delta_mixer)):
        m = cfg["layers"][i]["mixer"]
        NK, R = m["heads"] * m["dim"], m["rank"]
        w = {n: rand(NK, W, seed=10 + j, scale=0.2).double() for j, n in enumerate("rkvga")}
        w.update({"w1": rand(R, W, seed=20).double(), "w2": rand(NK, R, seed=21).double(), "w0": rand(NK, seed=22).double(),
                  "norm": 1 + rand(NK, seed=23, scale=0.1).double(), "o": rand(W, NK, seed=24, scale=0.2).double(),
                  "u": rand(m["heads"], m["dim"], seed=25).double(), "a.b": rand(NK, seed=26).double()})
        w.update({"mu." + s: torch.rand(W, generator=torch.Generator().manual_seed(30 + j)).double() for j, s in enumerate("rkvgw")})
        full = fn(x, w, m, 1e-5)
        assert torch.allclose(fn(x[:7], w, m, 1e-5), full[:7], atol=1e-12)
        assert torch.isfinite(full).all() and float(full.abs().max()) > 1e-3
