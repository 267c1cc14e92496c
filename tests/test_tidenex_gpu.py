"""The Tidenex design in the engine against the plain implementation: each mechanism alone, then whole models under
every way of cutting and batching, long decoding, generation through the scheduler, and the trace replay."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import schedules
from helpers import TOL, assert_greedy_follows_plain, max_rel_err, random_tokens
from plain import tidenex as PT
from test_engine_gpu import first_bad, run_schedule
from test_zatupel_gpu import CUTS, DEV, DT, DTYPES, PART_TOL, _bf16_weights, _feed, _rt, make_runner
from tidenex_models import LENGTHS, TID, make_tid_dir
from zatupel_models import rand

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# ----------------------------------------------------------------------------------------------- small kernels

@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("H", [7, 48, 1030])
def test_layer_norm(dtype, H):
    from forge_b200 import kernels
    x = (rand(9, H, seed=H, scale=3.0) + 5.0).to(DEV)                    # a mean far from zero
    w, b = (1.0 + rand(H, seed=1, scale=0.3)).to(DEV), rand(H, seed=2).to(DEV)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    want = PT.layer_norm(x.double().cpu(), w.double().cpu(), b.double().cpu(), 1e-3)
    assert max_rel_err(kernels.layernorm(x, w, b, 1e-3, dtype), want) <= PART_TOL[dtype]
    assert max_rel_err(kernels.layernorm(x, w, b, 1e-3, dtype, rows=rows), want[[8, 0, 3]]) <= PART_TOL[dtype]


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("W, I", [(48, 136), (256, 384)])
def test_dense_feed_forward(dtype, W, I):
    from forge_b200.config import PartSpec
    from forge_b200.parts import build_part
    ff = build_part("feed_forward", PartSpec("dense", {"hidden_size": W, "intermediate_size": I, "activation": "gelu"}), _rt(dtype))
    t = {n: rand(*s.shape, seed=i, scale=0.3).to(torch.bfloat16) for i, (n, s) in enumerate(ff.tensor_specs().items())}
    ff.bind(t)
    x = rand(19, W, seed=9, scale=1.5).to(dtype)
    r0 = rand(19, W, seed=10)
    res = r0.clone().to(DEV)
    ff.forward(x.to(DEV), res)
    want = r0.double() + PT.dense_ff(x.double(), t["mlp.up"].double(), t["mlp.down"].double())
    assert max_rel_err(res, want) <= PART_TOL[dtype]


def test_embedding_added_to_a_stream():
    from forge_b200 import kernels
    table = rand(20, 12).to(torch.bfloat16).to(DEV)
    ids = torch.tensor([3, 19, 0], dtype=torch.int32, device=DEV)
    x = rand(3, 12, seed=4).to(DEV)
    want = x.cpu() + table.float().cpu()[[3, 19, 0]]
    kernels.embedding(ids, table, out=x, add=True)
    assert torch.equal(x.cpu(), want)


# ----------------------------------------------------------------------------------------------- mixers alone

DIFFERENTIAL = {
    "values_not_two_maps_wide": dict(num_heads=6, num_kv_heads=3, head_dim=16, v_head_dim=24, scale=0.3, diff=0.35, rot=8, theta=300.0),
    "one_kv_head_whole_rotation": dict(num_heads=3, num_kv_heads=1, head_dim=8, v_head_dim=16, scale=0.5, diff=0.8, rot=8, theta=10000.0),
    "as_many_kv_heads_no_rotation_no_difference": dict(num_heads=2, num_kv_heads=2, head_dim=24, v_head_dim=8, scale=0.2, diff=0.0, rot=0, theta=10.0),
    "wide": dict(num_heads=8, num_kv_heads=2, head_dim=32, v_head_dim=64, scale=0.18, diff=0.4, rot=16, theta=1e6, out_scale=0.7,
                 tokens=150, cuts=[(0, 64), (64, 130), (130, 131), (131, 133), (133, 150)]),
}


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("kind", list(DIFFERENTIAL))
def test_differential_attention_alone(dtype, kind):
    from forge_b200.cache import CacheStorage
    from forge_b200.config import PartSpec
    from forge_b200.parts import build_part
    o = dict(DIFFERENTIAL[kind])
    W, T, cuts = 40, o.pop("tokens", 62), o.pop("cuts", CUTS)
    rot, theta = o.pop("rot"), o.pop("theta")
    spec = PartSpec("differential_attention", dict(o, hidden_size=W, eps=1e-4, position=PartSpec(
        "rope_halves", {"head_dim": o["head_dim"], "rotary_dims": rot, "theta": theta})))
    mixer = build_part("mixer", spec, _rt(dtype))
    t, w = _bf16_weights(mixer, 0.35, seed=len(kind))
    mixer.bind(t)
    storage = CacheStorage([mixer.cache_spec()], [None], 8, 48, 2, dtype, torch.device(DEV))
    x = rand(T, W, seed=50).to(dtype)
    got = _feed(mixer, storage, x, cuts, requests=("a", "b"))
    m = {"heads": o["num_heads"], "kv_heads": o["num_kv_heads"], "dim": o["head_dim"], "vdim": o["v_head_dim"], "scale": o["scale"],
         "diff": o["diff"], "rot": {"base": theta, "dims": rot}}
    want = PT.differential_attention(x.double(), w, m, 1e-4) * o.get("out_scale", 1.0)
    for r in ("a", "b"):
        assert max_rel_err(got[r], want) <= PART_TOL[dtype], (kind, r)


DISTANCE = {
    "one_kv_head": dict(num_heads=4, num_kv_heads=1, head_dim=24, v_head_dim=8, scale=0.2, temp_coef=0.5, temp_every=7.0, out_scale=1.3),
    "temperature_every_token": dict(num_heads=2, num_kv_heads=2, head_dim=16, v_head_dim=16, scale=0.25, temp_coef=0.2, temp_every=1.0),
    "no_temperature": dict(num_heads=3, num_kv_heads=3, head_dim=8, v_head_dim=40, scale=0.5),
}


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("kind", list(DISTANCE))
def test_distance_attention_alone(dtype, kind):
    from forge_b200.cache import CacheStorage
    from forge_b200.config import PartSpec
    from forge_b200.parts import build_part
    o = dict(DISTANCE[kind])
    W, T = 40, 62
    mixer = build_part("mixer", PartSpec("distance_attention", dict(o, hidden_size=W, eps=1e-3)), _rt(dtype))
    t, w = _bf16_weights(mixer, 0.35, seed=len(kind))
    mixer.bind(t)
    storage = CacheStorage([mixer.cache_spec()], [None], 8, 48, 2, dtype, torch.device(DEV))
    x = rand(T, W, seed=51).to(dtype)
    got = _feed(mixer, storage, x, CUTS, requests=("a", "b"))
    m = {"heads": o["num_heads"], "kv_heads": o["num_kv_heads"], "dim": o["head_dim"], "vdim": o["v_head_dim"], "scale": o["scale"],
         "q_temp": {"coef": o.get("temp_coef", 0.0), "every": o.get("temp_every", 1.0)}}
    want = PT.biased_attention(x.double(), w, m, 1e-3) * o.get("out_scale", 1.0)
    for r in ("a", "b"):
        assert max_rel_err(got[r], want) <= PART_TOL[dtype], (kind, r)


GATED = [(3, 10, 6), (2, 6, 10), (5, 12, 20), (1, 40, 24), (4, 64, 32), (2, 32, 64), (2, 128, 16), (1, 8, 130), (1, 160, 8), (2, 256, 24)]


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("heads, dim, vdim", GATED)
def test_gated_write_alone(dtype, heads, dim, vdim):
    from forge_b200.cache import CacheStorage
    from forge_b200.config import PartSpec
    from forge_b200.parts import build_part
    W, T, eps = 56, 62, 1e-4
    mixer = build_part("mixer", PartSpec("gated_write", {"hidden_size": W, "num_heads": heads, "head_dim": dim, "v_head_dim": vdim,
                                                         "eps": eps, "out_scale": 1.1}), _rt(dtype))
    t, w = _bf16_weights(mixer, 0.25, seed=heads + dim)
    mixer.bind(t)
    storage = CacheStorage([mixer.cache_spec()], [None], 8, 8, 3, dtype, torch.device(DEV))
    x = rand(T, W, seed=60).to(dtype)
    # a slot that another request used before: its rows must come back as zeros
    _feed(mixer, storage, x, [(0, 9)], requests=("old",))
    storage.manager.free("old")
    got = _feed(mixer, storage, x, CUTS, requests=("a", "b"))
    want, _ = PT.gated_linear_recurrence(x.double(), w, {"heads": heads, "dim": dim, "vdim": vdim}, eps)
    for r in ("a", "b"):
        assert max_rel_err(got[r], want * 1.1) <= PART_TOL[dtype], r


@pytest.mark.parametrize("dtype", DT)
def test_a_state_that_is_lost_shows(dtype):
    """A forget gate held near one by its lower bound: what the first token wrote is still most of the output 60 tokens later, so
    a state that was dropped or zeroed between steps could not pass."""
    from forge_b200.cache import CacheStorage
    from forge_b200.config import PartSpec
    from forge_b200.parts import build_part
    W, T = 32, 61
    mixer = build_part("mixer", PartSpec("gated_write", {"hidden_size": W, "num_heads": 2, "head_dim": 8, "v_head_dim": 8, "eps": 1e-5}), _rt(dtype))
    t, w = _bf16_weights(mixer, 0.25, seed=5)
    t["mix.lower"] = torch.full((16,), 0.996).to(torch.bfloat16)
    w["lower"] = t["mix.lower"].double()
    mixer.bind(t)
    storage = CacheStorage([mixer.cache_spec()], [None], 8, 8, 2, dtype, torch.device(DEV))
    x = rand(T, W, seed=61).to(dtype)
    x[1:] *= 0.05                                                          # later tokens write little
    got = _feed(mixer, storage, x, [(0, 1)] + [(i, i + 1) for i in range(1, 40)] + [(40, 61)])["r"]
    m = {"heads": 2, "dim": 8, "vdim": 8}
    want, _ = PT.gated_linear_recurrence(x.double(), w, m, 1e-5)
    lost, _ = PT.gated_linear_recurrence(x.double()[1:], w, m, 1e-5)
    assert max_rel_err(got, want) <= PART_TOL[dtype]
    assert max_rel_err(lost, want[1:]) > 0.3                               # the test would see it


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("rv", [4, 5])       # 5: an odd number of output columns in all, so the two mixers keep products of their own
def test_side_by_side_mixers_in_a_layer(dtype, rv):
    """A whole pre-norm layer whose mixer is an attention beside a recurrence: pages and a state row behind one layer, one
    input product and one output product for both mixers."""
    from forge_b200.cache import CacheStorage
    from forge_b200.config import LayerSpec, PartSpec
    from forge_b200.engine import StepEntry, build_step_batch
    from forge_b200.parts import build_block
    W, T, eps = 48, 37, 1e-3
    norm = lambda n: PartSpec("layernorm", {"size": W, "eps": eps, "names": {"weight": n, "bias": n + ".b"}})
    mixer = PartSpec("side_by_side", {"mixers": [
        PartSpec("distance_attention", {"hidden_size": W, "num_heads": 4, "num_kv_heads": 2, "head_dim": 8, "v_head_dim": 12, "scale": 0.3,
                                        "eps": eps, "temp_coef": 0.4, "temp_every": 5.0, "out_scale": 0.6, "prefix": "mix.left."}),
        PartSpec("gated_write", {"hidden_size": W, "num_heads": 3, "head_dim": 8, "v_head_dim": rv, "eps": eps, "out_scale": 1.7,
                                 "prefix": "mix.right."})]})
    spec = LayerSpec(block="pre_norm", mixer=mixer, feed_forward=PartSpec("dense", {"hidden_size": W, "intermediate_size": 72}),
                     norms={"input": norm("norm1"), "post_mixer": norm("norm2")}, weight_prefix="", norm_prefixes={"input": "", "post_mixer": ""})
    block = build_block(spec, _rt(dtype))
    bt, _ = _bf16_weights(block, 0.25, seed=3)
    block.bind(bt)
    assert (block.mixer.proj is not None) == (rv == 4)
    storage = CacheStorage([block.mixer.cache_spec()], [None], 8, 8, 1, dtype, torch.device(DEV))
    assert len(storage.layers[0].parts) == 2 and storage.layers[0].parts[0].kv is not None and storage.layers[0].parts[1].state is not None
    storage.manager.admit("r")
    r0 = rand(T, W, seed=12)
    res = r0.clone().to(DEV)
    for a, b in ((0, 20), (20, 21), (21, 37)):
        batch = build_step_batch([StepEntry("r", [0] * (b - a), [])], storage.manager, torch.device(DEV), 8)
        storage.zero_state_slots(storage.manager.take_fresh_slots())
        part = res[a:b].contiguous()
        block.forward(part, batch, storage.layers[0])
        res[a:b] = part
    d = {k: v.double() for k, v in bt.items()}
    mw = {k.split("mix.", 1)[1]: v for k, v in d.items() if k.startswith("mix.")}
    m = {"left": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.3, "q_temp": {"coef": 0.4, "every": 5}},
         "right": {"heads": 3, "dim": 8, "vdim": rv}, "left_scale": 0.6, "right_scale": 1.7}
    x = r0.double()
    x = x + PT.parallel_mixer(PT.layer_norm(x, d["norm1"], d["norm1.b"], eps), mw, m, eps)
    want = x + PT.dense_ff(PT.layer_norm(x, d["norm2"], d["norm2.b"], eps), d["mlp.up"], d["mlp.down"])
    assert max_rel_err(res, want) <= PART_TOL[dtype]


# ----------------------------------------------------------------------------------------------- keys that stand out

@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("page_size", [8, 64])
@pytest.mark.parametrize("maps", [1, 2])
@pytest.mark.parametrize("D, E", [(8, 2), (16, 8)])          # the second pair is one that the tensor-core kernel takes in bfloat16
def test_one_key_that_stands_out(dtype, page_size, maps, D, E):
    """Keys are zero except one whose score is huge for head 0's first map; values carry their position.  That map returns the
    key's position if the token sees it (far back among hundreds, at a page's border, the token itself) and the mean of the
    visible positions if it does not (the key lies ahead, in the same portion); every other map returns the mean.  With two
    maps the result is (a_1 - lambda a_2) over its root mean square.  For a prompt's portion and for single tokens."""
    from forge_b200 import kernels
    from forge_b200.cache import CacheStorage
    from forge_b200.engine import StepEntry, build_step_batch
    from forge_b200.parts import KVCacheSpec
    H, G, N, P = 2, 1, 300, 27
    lam, post, eps = 0.4, 0.7, 1e-6
    dev = torch.device(DEV)
    storage = CacheStorage([KVCacheSpec(G, maps * D, None, v_head_dim=E)], [None], page_size, 64 * 8 // page_size, 2, dtype, dev)
    group = next(iter(storage.manager.groups))
    QW, KW = H * maps * D, G * maps * D
    for case, star in enumerate([0, 150, 63, 64, N - 1, N, N + 5, N + P - 1, N + P, N + P + 1]):
        rid = f"r{case}"
        storage.manager.admit(rid)
        total = N + P + 2
        proj = torch.zeros(total, QW + KW + G * E)
        proj[:, 0] = 10.0                                                  # head 0, map 1 asks for the key; the others for nothing
        proj[star, QW] = 10.0                                              # the key that stands out (in map 1's channels)
        proj[:, QW + KW] = torch.arange(total, dtype=torch.float32)        # a value's first channel: its position
        proj[:, QW + KW + 1] = 1.0
        done = 0
        for n in (N, P, 1, 1):                                             # the context, a portion, two single tokens
            batch = build_step_batch([StepEntry(rid, [0] * n, [])], storage.manager, dev, 64)
            g = batch.groups[group]
            rows = proj[done:done + n].to(DEV).contiguous()
            q = kernels.scored_prepare(rows, batch.positions, g.slot_mapping, storage.layers[0].kv, H, G, maps, D, E, page_size, dtype)
            out = kernels.scored_attention(q, storage.layers[0].kv, g, batch, H, G, maps, D, E, page_size, 1.0, lam=lam, post=post,
                                           eps=eps).float().cpu().view(n, H, E)
            for t in range(n) if n <= P else ():
                i = done + t
                mean = i / 2.0
                a1 = float(star) if star <= i else mean
                tol = 1e-4 if dtype == torch.float32 else 2e-2
                for h, first in ((0, a1), (1, mean)):
                    if maps == 1:
                        want = [first, 1.0]
                    else:
                        o = [first - lam * mean, 1.0 - lam]
                        rms = math.sqrt((o[0] ** 2 + o[1] ** 2) / E + eps)          # the other value channels are zero
                        want = [o[0] / rms * post, o[1] / rms * post]
                    scale = max(1.0, abs(want[0]))
                    assert abs(out[t, h, 0] - want[0]) <= tol * scale and abs(out[t, h, 1] - want[1]) <= tol * scale, \
                        (star, i, h, out[t, h].tolist(), want)
            done += n
        storage.manager.free(rid)                                          # the next case takes over these pages
        storage.manager.check()


@pytest.mark.parametrize("dtype", DT)
def test_distance_term_counts_from_the_token(dtype):
    """Zero queries: a head's weights are (1 + r2 d)^(-r1) over the distance d to the key, whatever the portion or the page;
    head 1 has r1 = 0 and returns the mean."""
    from forge_b200 import kernels
    from forge_b200.cache import CacheStorage
    from forge_b200.engine import StepEntry, build_step_batch
    from forge_b200.parts import KVCacheSpec
    H, G, D, E, N, P, page_size = 2, 1, 8, 2, 200, 19, 8
    dev = torch.device(DEV)
    storage = CacheStorage([KVCacheSpec(G, D, None, v_head_dim=E)], [None], page_size, 32, 1, dtype, dev)
    group = next(iter(storage.manager.groups))
    r1, r2 = torch.tensor([2.0, 0.0], device=DEV), torch.tensor([0.5, 3.0], device=DEV)
    total = N + P + 1
    proj = torch.zeros(total, (H + G) * D + G * E)
    proj[:, (H + G) * D] = torch.arange(total, dtype=torch.float32)
    proj[:, (H + G) * D + 1] = 1.0
    storage.manager.admit("r")
    done = 0
    for n in (N, P, 1):
        batch = build_step_batch([StepEntry("r", [0] * n, [])], storage.manager, dev, 64)
        g = batch.groups[group]
        q = kernels.scored_prepare(proj[done:done + n].to(DEV).contiguous(), batch.positions, g.slot_mapping, storage.layers[0].kv, H, G, 1,
                                   D, E, page_size, dtype)
        out = kernels.scored_attention(q, storage.layers[0].kv, g, batch, H, G, 1, D, E, page_size, 1.0, r1=r1, r2=r2).float().cpu().view(n, H, E)
        for t in range(n) if n <= P else ():
            i = done + t
            wt = [(1 + 0.5 * (i - j)) ** -2.0 for j in range(i + 1)]
            near = sum(w * j for w, j in zip(wt, range(i + 1))) / sum(wt)
            tol = (1e-4 if dtype == torch.float32 else 2e-2) * i
            assert abs(out[t, 0, 0] - near) <= tol and abs(out[t, 1, 0] - i / 2.0) <= tol, (i, out[t, :, 0].tolist(), near)
        done += n


@pytest.mark.parametrize("dtype", DT)
def test_prepare_norms_rotates_and_heats(dtype):
    """The prepare step alone: the norm over all of q (and of k) with its weights, the rotation of every map's first channels
    with the pair half the rotated width apart, and the temperature, against the plain functions."""
    from forge_b200 import kernels
    from forge_b200.cache import CacheStorage
    from forge_b200.engine import StepEntry, build_step_batch
    from forge_b200.parts import KVCacheSpec
    H, G, M, D, E, T, page_size = 3, 1, 2, 12, 4, 45, 8
    dev = torch.device(DEV)
    storage = CacheStorage([KVCacheSpec(G, M * D, None, v_head_dim=E)], [None], page_size, 8, 1, dtype, dev)
    storage.manager.admit("r")
    batch = build_step_batch([StepEntry("r", [0] * T, [])], storage.manager, dev, 64)
    g = batch.groups[next(iter(storage.manager.groups))]
    proj = rand(T, (H + G) * M * D + G * E, seed=70)
    qn, kn = 1.0 + rand(H * M * D, seed=71, scale=0.3), 1.0 + rand(G * M * D, seed=72, scale=0.3)
    freq = torch.pow(torch.tensor(40.0, dtype=torch.float64), -2.0 * torch.arange(3, dtype=torch.float64) / 6).float().to(DEV)
    q = kernels.scored_prepare(proj.to(DEV), batch.positions, g.slot_mapping, storage.layers[0].kv, H, G, M, D, E, page_size, dtype, inv_freq=freq,
                               q_norm=qn.to(DEV), k_norm=kn.to(DEV), eps=1e-3, temp_coef=0.6, temp_every=4.0)
    pos = torch.arange(T)
    pq = PT.rms_unit(proj[:, :H * M * D].double(), 1e-3) * qn.double()
    pq = PT.rotate_halves(pq.view(T, H * M, D), pos, 40.0, 6).reshape(T, -1)
    temp = 1.0 + 0.6 * torch.log(torch.floor((pos.double() + 1) / 4.0) + 1.0)
    assert max_rel_err(q, pq * temp[:, None]) <= PART_TOL[dtype]
    pk = PT.rms_unit(proj[:, H * M * D:(H + G) * M * D].double(), 1e-3) * kn.double()
    pk = PT.rotate_halves(pk.view(T, G * M, D), pos, 40.0, 6).reshape(T, G, M * D)
    table = storage.manager.block_table("r", next(iter(storage.manager.groups)))
    kv = storage.layers[0].kv.reshape(storage.layers[0].kv.shape[0], -1).float().cpu()
    for t in (0, 7, 8, 44):
        page = kv[table[t // page_size]]
        keys = page[:G * page_size * M * D].view(G, page_size, M * D)[:, t % page_size]
        vals = page[G * page_size * M * D:].view(G, page_size, E)[:, t % page_size]
        assert max_rel_err(keys, pk[t]) <= PART_TOL[dtype]
        assert max_rel_err(vals, proj[t, (H + G) * M * D:].view(G, E)) <= PART_TOL[dtype]


# ----------------------------------------------------------------------------------------------- whole models

@pytest.fixture(scope="module", params=["X", "Y", "Z"])
def tid(request, tmp_path_factory):
    name = request.param
    d = make_tid_dir(tmp_path_factory, name)
    plain = PT.PlainTidenex.from_dir(d)
    reqs = {f"r{i}": random_tokens(n, TID[name]["vocab"], seed=10 * i + ord(name)) for i, n in enumerate(LENGTHS[name])}
    want = {rid: plain.forward(toks).float() for rid, toks in reqs.items()}
    return name, d, plain, reqs, want


def test_layer_by_layer(tid):
    """The residual stream after every run of a layer (a repeated layer counts each time), in 32-bit."""
    name, d, plain, reqs, want = tid
    from forge_b200.engine import StepEntry
    runner = make_runner(d, "float32", 256)
    streams = []
    for b in set(runner.model.blocks):
        def wrap(orig):
            def f(residual, batch, cache):
                orig(residual, batch, cache)
                streams.append(residual.clone())
            return f
        b.forward = wrap(b.forward)
    toks = reqs["r2"]
    runner.admit("x")
    runner.step([StepEntry("x", toks, [])])
    _, ref = plain.forward(toks, keep_layers=True)
    assert len(streams) == ref.shape[0]
    for i, s in enumerate(streams):
        assert max_rel_err(s, ref[i]) <= 2e-5, f"run {i} of the schedule"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("schedule", ["whole", "last_one_by_one", "changing_portions", "mixed"])
def test_schedules_equal_plain(tid, dtype, schedule):
    name, d, plain, reqs, want = tid
    steps = getattr(schedules, schedule)(reqs)
    # exactly as many pages as the schedule's peak needs: freed pages and slots are taken again at once
    runner = make_runner(d, dtype, schedules.peak_tokens(reqs, steps, round_to=8))
    got = run_schedule(runner, reqs, steps)
    assert first_bad(got, want, TOL[dtype]) is None, first_bad(got, want, TOL[dtype])
    assert runner.manager.num_free_pages() == {g: runner.num_pages for g in runner.manager.groups}


@pytest.mark.parametrize("dtype", DTYPES)
def test_page_size_and_graphs_do_not_matter(tid, dtype):
    name, d, plain, reqs, want = tid
    small = {k: reqs[k] for k in list(reqs)[:3]}
    for ps, graphs in ((16, True), (64, True), (8, False)):
        steps = schedules.mixed(small, max_live=2)
        runner = make_runner(d, dtype, schedules.peak_tokens(small, steps, round_to=ps), page_size=ps, cuda_graphs=graphs)
        got = run_schedule(runner, small, steps)
        msg = first_bad(got, {k: want[k] for k in small}, TOL[dtype])
        assert msg is None, f"page size {ps}: {msg}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_and_first_tokens(tid, dtype):
    """Two tokens, one, then hundreds one by one: the state runs long, the temperature steps up, pages fill and follow."""
    name, d, plain, reqs, want = tid
    n = {"X": 230, "Y": 260, "Z": 170}[name]
    toks = random_tokens(n, TID[name]["vocab"], seed=77)
    ref = plain.forward(toks).float()
    runner = make_runner(d, dtype, -(-n // 8) * 8)
    steps = [([("x", 0, 2)], [])] + [([("x", p, 1)], []) for p in range(2, n)]
    got = run_schedule(runner, {"x": toks}, steps)
    msg = first_bad(got, {"x": ref}, TOL[dtype])
    assert msg is None, msg


def test_fp32_logits_do_not_depend_on_the_cut(tid):
    """In 32-bit every sum is taken in an order that the position alone decides: the four schedules agree to rounding."""
    name, d, plain, reqs, want = tid
    small = {k: reqs[k] for k in list(reqs)[:3]}
    outs = []
    for schedule in ("whole", "last_one_by_one", "changing_portions", "mixed"):
        steps = getattr(schedules, schedule)(small)
        runner = make_runner(d, "float32", schedules.peak_tokens(small, steps, round_to=8), cuda_graphs=False)
        outs.append(run_schedule(runner, small, steps))
    for o in outs[1:]:
        for rid in small:
            assert float((o[rid] - outs[0][rid]).abs().max()) <= 2e-5 * float(outs[0][rid].abs().max()), rid


@pytest.mark.parametrize("dtype", DTYPES)
def test_generation_through_the_scheduler(tid, dtype):
    """Greedy generation through forge.Model and through RequestScheduler with more requests than slots and few pages."""
    import forge_b200 as forge
    name, d, plain, reqs, want = tid
    model = forge.Model(d, dtype=dtype, block_size=8, max_num_seqs=2, cache_tokens=512, max_tokens_per_step=48)
    prompt = reqs["r1"][:37]
    out = model.generate(prompt, max_new_tokens=12, do_sample=False)
    assert out["num_generated_tokens"] == 12 and out["finish_reason"] == "length"
    logits_fn = lambda ids: plain.forward(ids).float()
    assert_greedy_follows_plain(logits_fn, prompt, out["token_ids"], TOL[dtype], what="generate")
    sched = forge.RequestScheduler(model, max_num_seqs=2, max_tokens_per_step=48)
    prompts = [reqs["r0"][:50], reqs["r2"][:9], reqs["r3"][:31], reqs["r1"][:3]]
    ids = [sched.submit(p, 8, -1, forge.SamplerConfig(do_sample=False)) for p in prompts]
    done = {r.request_id: r for r in sched.run()}
    for rid, p in zip(ids, prompts):
        assert done[rid].num_generated == 8
        assert_greedy_follows_plain(logits_fn, p, list(done[rid].output_tokens), TOL[dtype], what=f"request {rid}")
    model.runner.manager.check()
    model.runner.check_status()


def test_trace_replay_as_a_subprocess(tid, tmp_path):
    name, d, plain, reqs, want = tid
    small = {k: reqs[k] for k in list(reqs)[:3]}
    steps = schedules.mixed(small, max_live=2)
    lines, asked = [], {}
    for n, (entries, end) in enumerate(steps):
        es = []
        for rid, p, cnt in entries:
            w = [cnt - 1] if (p + cnt) % 3 == 0 or p + cnt == len(small[rid]) else []
            es.append({"id": rid, "tokens": small[rid][p:p + cnt], "want": w})
            if w:
                asked.setdefault(n, []).extend((rid, p + i) for i in w)
        lines.append(json.dumps({"step": n, "entries": es, "end": end}))
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", str(out),
                        "--max-tokens", str(schedules.peak_tokens(small, steps, round_to=64))], input="\n".join(lines) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {n}" for n in range(len(steps))]
    V = TID[name]["vocab"]
    for n, rows in asked.items():
        got = torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(len(rows), V))
        ref = torch.stack([want[rid][pos] for rid, pos in rows])
        assert max_rel_err(got, ref) <= TOL["float32"], n
    assert sorted(os.listdir(out)) == sorted(f"{n}.f32" for n in asked)


def test_command_line(tid):
    """bin/forge-cli on a Tidenex folder: greedy tokens in 32-bit follow the plain implementation; sampling runs."""
    name, d, plain, reqs, want = tid
    prompt = reqs["r1"][:6]
    cli = [sys.executable, os.path.join(ROOT, "bin", "forge-cli"), "-m", d, "-p", " ".join(map(str, prompt)), "-n", "5", "--no-stream",
           "--page-size", "8", "--kv-pages", "2"]
    proc = subprocess.run(cli + ["--temp", "0", "--repeat-penalty", "1.0", "--dtype", "float32"], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = [int(t) for t in proc.stdout.strip().splitlines()[0].split()]
    assert len(got) == 5 and "6 prompt" in proc.stdout and "5 generated" in proc.stdout
    assert_greedy_follows_plain(lambda ids: plain.forward(ids).float(), prompt, got, TOL["float32"], what="forge-cli")
    proc = subprocess.run(cli + ["--temp", "0.8", "--top-k", "20", "--seed", "3", "--dtype", "bfloat16"], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert len(proc.stdout.strip().splitlines()[0].split()) == 5
