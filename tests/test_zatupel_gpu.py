"""The Zatupel design in the engine against the plain implementation: each mechanism alone, then whole models under
every way of cutting and batching, long decoding, generation through the scheduler, and the trace replay."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import schedules
from helpers import TOL, assert_greedy_follows_plain, max_rel_err, random_tokens
from plain import zatupel as PZ
from test_engine_gpu import first_bad, run_schedule
from zatupel_models import LENGTHS, ZAT, make_zat_dir, rand

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
DT = [torch.float32, torch.bfloat16]
PART_TOL = {torch.float32: 2e-5, torch.bfloat16: 3e-2}


def _rt(dtype):
    from forge_b200.parts import Runtime
    return Runtime(torch.device(DEV), dtype)


def _bf16_weights(part, std, seed=0):
    """Random tensors for a part, as a file would hold them (bfloat16), and the same numbers in float64."""
    t = {}
    for i, (n, s) in enumerate(part.tensor_specs().items()):
        shape = s.default_shape if -1 in s.shape else s.shape
        if s.role == "fraction":
            x = torch.rand(shape, generator=torch.Generator().manual_seed(seed + i))
        elif s.role == "norm":
            x = 1.0 + rand(*shape, seed=seed + i, scale=0.2)
        elif s.role == "head_mix":
            x = torch.eye(shape[0]) + rand(*shape, seed=seed + i, scale=0.4)
        elif s.role == "bias":
            x = rand(*shape, seed=seed + i, scale=0.7)
        else:
            x = rand(*shape, seed=seed + i, scale=std)
        t[n] = x.to(torch.bfloat16)
    return t, {n.split("mix.", 1)[-1]: v.double() for n, v in t.items()}


def _feed(mixer, storage, x, cuts, requests=("r",), shared=None):
    """Feeds x [T, W] (the same for every request) through the mixer in the given portions, every request in the same
    step; returns {request: [T, W]} of what the mixer added to a zero residual."""
    from forge_b200.engine import StepEntry, build_step_batch
    T, W = x.shape
    got = {r: torch.zeros(T, W) for r in requests}
    for r in requests:
        storage.manager.admit(r)
    for a, b in cuts:
        batch = build_step_batch([StepEntry(r, [0] * (b - a), []) for r in requests], storage.manager, torch.device(DEV), 64)
        storage.zero_state_slots(storage.manager.take_fresh_slots())
        if shared is not None:
            batch.shared.update({k: torch.cat([v[a:b]] * len(requests)).to(DEV).contiguous() for k, v in shared.items()})
        res = torch.zeros(len(requests) * (b - a), W, device=DEV)
        mixer.forward(torch.cat([x[a:b]] * len(requests)).to(DEV).contiguous(), batch, storage.layers[0], res)
        for i, r in enumerate(requests):
            got[r][a:b] = res[i * (b - a):(i + 1) * (b - a)].cpu()
            storage.manager.release_out_of_window(r)
        storage.manager.check()
    return got


CUTS = [(0, 13), (13, 28), (28, 29), (29, 31), (31, 32), (32, 61), (61, 62)]

ATTENTIONS = {
    "everything": dict(num_heads=6, num_kv_heads=2, head_dim=24, v_head_dim=8, scale=0.31, window=9, keep_first=3, rot=16, theta=300.0),
    "plain_gqa": dict(num_heads=4, num_kv_heads=4, head_dim=16, v_head_dim=16, scale=None, window=None, keep_first=0, rot=16, theta=10000.0,
                      head_mix=False, head_gate=False),
    "one_kv_head_no_rotation": dict(num_heads=3, num_kv_heads=1, head_dim=8, v_head_dim=40, scale=0.5, window=30, keep_first=0, rot=0,
                                    theta=10.0, head_gate=False),
    # more kept first tokens than a key tile holds, and a window far behind them: 150 tokens in other portions
    "many_kept": dict(num_heads=4, num_kv_heads=2, head_dim=16, v_head_dim=8, scale=0.4, window=11, keep_first=70, rot=16, theta=50.0,
                      tokens=150, cuts=[(0, 64), (64, 130), (130, 131), (131, 133), (133, 150)]),
    # all key/value heads' values side by side make 128 and 256 columns: the tensor-core kernel's other two chunk widths
    "values_128_wide": dict(num_heads=4, num_kv_heads=2, head_dim=16, v_head_dim=64, scale=0.35, window=25, keep_first=2, rot=8, theta=900.0),
    "values_256_wide": dict(num_heads=4, num_kv_heads=4, head_dim=32, v_head_dim=64, scale=0.25, window=40, keep_first=0, rot=32, theta=1e4,
                            head_gate=False),
    "blend": dict(num_heads=2, num_kv_heads=2, head_dim=32, v_head_dim=16, scale=0.2, window=7, keep_first=7, rot=32, theta=77.0,
                  head_mix=False, value_mix="blend"),
}


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("kind", list(ATTENTIONS))
def test_attention_mixer_alone(dtype, kind):
    from forge_b200.cache import CacheStorage
    from forge_b200.config import PartSpec
    from forge_b200.parts import build_part
    o = dict(ATTENTIONS[kind])
    W, T, cuts = 40, o.pop("tokens", 62), o.pop("cuts", CUTS)
    rot, theta = o.pop("rot"), o.pop("theta")
    spec = PartSpec("headmix_attention", dict(o, hidden_size=W, position=PartSpec("rope_pairs", {"head_dim": o["head_dim"], "rotary_dims": rot,
                                                                                              "theta": theta})))
    mixer = build_part("mixer", spec, _rt(dtype))
    t, w = _bf16_weights(mixer, 0.35, seed=len(kind))
    mixer.bind(t)
    storage = CacheStorage([mixer.cache_spec()], [None], 8, 48, 2, dtype, torch.device(DEV))
    x = rand(T, W, seed=50).to(dtype)
    G, E = o["num_kv_heads"], o["v_head_dim"]
    v_first = rand(T, G * E, seed=51) if o.get("value_mix") == "blend" else None
    got = _feed(mixer, storage, x, cuts, requests=("a", "b"), shared=None if v_first is None else {"first_values": v_first})
    m = {"heads": o["num_heads"], "kv_heads": G, "dim": o["head_dim"], "vdim": E, "scale": mixer.scale,
         "mask": {"size": o["window"] or 10 ** 6, "keep_first": o["keep_first"]}, "rot": {"base": theta, "dims": rot}}
    w.setdefault("talk", torch.eye(o["num_heads"], dtype=torch.float64))
    if "g" not in w:
        w["g"] = torch.zeros(o["num_heads"], W, dtype=torch.float64)
    want, _ = PZ.attention_mixer(x.double(), torch.arange(T), w, m, None if v_first is None else v_first.double().view(T, G, E))
    if not o.get("head_gate", True):
        want = want * 2.0                       # the plain mixer always gates; a zero gate matrix halves
    for r in ("a", "b"):
        assert max_rel_err(got[r], want) <= PART_TOL[dtype], (kind, r)
    if kind == "everything":                     # 62 tokens, window 9, pages of 8: the pages between the kept first and the window are back
        table = storage.manager.block_table("a", next(iter(storage.manager.groups)))
        assert table[0] >= 0 and table[1:6] == [-1] * 5 and table[7] >= 0


def _visible(i, j, size, keep):
    return j <= i and (i - j < size or j < keep)


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("page_size", [8, 64])
@pytest.mark.parametrize("D, E", [(8, 4), (16, 8)])          # the second pair is one that the tensor-core kernel takes in bfloat16
def test_one_key_that_stands_out(dtype, page_size, D, E):
    """Keys are zero except one, far away among hundreds, at a window's edge or among the kept first, whose score is
    huge for head 0; values carry their position.  Head 0 (before the heads' exchange) returns that position if it is
    visible and the mean of the visible positions if it is not; head 1 always the mean.  For tokens of a prompt portion
    (whose window edges lie inside a tile and across page borders) and for single tokens."""
    from forge_b200 import kernels
    from forge_b200.cache import CacheStorage
    from forge_b200.engine import StepEntry, build_step_batch
    from forge_b200.parts import KVCacheSpec
    H, G, size, keep, N, M = 2, 1, 21, 3, 300, 27
    dev = torch.device(DEV)
    mix = torch.tensor([[0.7, 0.3], [0.2, 0.8]], device=DEV)
    storage = CacheStorage([KVCacheSpec(G, D, size, v_head_dim=E, keep_first=keep)], [None], page_size, 64 * 8 // page_size, 2, dtype, dev)
    group = next(iter(storage.manager.groups))
    none = torch.zeros(0, device=DEV)
    for case, star in enumerate([N - size + 1, N - size, N - size + 5, keep - 1, keep, 0, 150, N + 3, N - 1]):
        rid = f"r{case}"
        storage.manager.admit(rid)
        total = N + M + 2
        proj = torch.zeros(total, (H + G) * D + G * E)
        proj[star, H * D] = 10.0                                           # the key that stands out
        proj[:, (H + G) * D] = torch.arange(total, dtype=torch.float32)    # a value's first channel: its position
        proj[:, (H + G) * D + 1] = 1.0
        q = torch.zeros(total, H * D)
        q[:, 0] = 10.0                                                     # head 0 asks for it, head 1 for nothing
        done = 0
        for n in (N, M, 1, 1):                                            # the context, a portion, two single tokens
            batch = build_step_batch([StepEntry(rid, [0] * n, [])], storage.manager, dev, 64)
            g = batch.groups[group]
            rows = proj[done:done + n].to(DEV).contiguous()
            kernels.headmix_prepare(rows, batch.positions, g.slot_mapping, none, storage.layers[0].kv, H, G, D, E, page_size, dtype, has_gate=False)
            out = kernels.headmix_attention(q[done:done + n].to(DEV).to(dtype).contiguous(), storage.layers[0].kv, g, batch, H, G, D, E,
                                            page_size, 1.0, window=size, keep_first=keep, mix=mix).float().cpu().view(n, H, E)
            for t in range(n) if n <= M else ():
                i = done + t
                seen = [j for j in range(i + 1) if _visible(i, j, size, keep)]
                mean = sum(seen) / len(seen)
                head0 = float(star) if star in seen else mean
                want = [0.7 * head0 + 0.3 * mean, 0.2 * head0 + 0.8 * mean]
                tol = 1e-4 * i if dtype == torch.float32 else 2e-2 * i
                assert abs(out[t, 0, 0] - want[0]) <= tol and abs(out[t, 1, 0] - want[1]) <= tol, (star, i, out[t, :, 0].tolist(), want)
                assert abs(out[t, 0, 1] - 1.0) <= 1e-2 and abs(out[t, 1, 1] - 1.0) <= 1e-2      # the weights add up to one
            done += n
            storage.manager.release_out_of_window(rid)
        storage.manager.free(rid)                                          # the next case takes over these pages
        storage.manager.check()


STATE_MIXERS = [("wkv", 3, 10, 4), ("general_delta", 2, 6, 4),          # channels that are no multiple of four: staged one by one
                ("wkv", 5, 16, 8), ("wkv", 1, 40, 24), ("wkv", 2, 64, 4), ("general_delta", 3, 24, 12), ("general_delta", 4, 8, 16),
                ("general_delta", 1, 96, 8), ("wkv", 2, 128, 8), ("general_delta", 2, 128, 8)]


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("kind, heads, dim, rank", STATE_MIXERS)
def test_state_mixer_alone(dtype, kind, heads, dim, rank):
    from forge_b200.cache import CacheStorage
    from forge_b200.config import PartSpec
    from forge_b200.parts import build_part
    W, T, eps = 56, 62, 1e-4
    mixer = build_part("mixer", PartSpec(kind, {"hidden_size": W, "num_heads": heads, "head_dim": dim, "eps": eps, "rank": rank}), _rt(dtype))
    t, w = _bf16_weights(mixer, 0.25, seed=heads + dim)
    mixer.bind(t)
    storage = CacheStorage([mixer.cache_spec()], [None], 8, 8, 3, dtype, torch.device(DEV))
    x = rand(T, W, seed=60).to(dtype)
    # a slot that another request used before: its rows must come back as zeros
    _feed(mixer, storage, x, [(0, 9)], requests=("old",))
    storage.manager.free("old")
    got = _feed(mixer, storage, x, CUTS, requests=("a", "b"))
    fn = PZ.wkv_mixer if kind == "wkv" else PZ.general_delta_mixer
    want = fn(x.double(), w, {"heads": heads, "dim": dim}, eps)
    for r in ("a", "b"):
        assert max_rel_err(got[r], want) <= PART_TOL[dtype], (kind, r)


@pytest.mark.parametrize("dtype", DT)
def test_gated_gelu_and_parallel_block(dtype):
    """The feed-forward alone, then a whole layer: both branches read the residual stream as the layer found it."""
    from forge_b200.cache import CacheStorage
    from forge_b200.config import LayerSpec, PartSpec
    from forge_b200.engine import StepEntry, build_step_batch
    from forge_b200.parts import build_block, build_part
    W, I, T = 48, 136, 19
    names = {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}
    ff_spec = PartSpec("geglu", {"hidden_size": W, "intermediate_size": I, "suffix": "", "names": names})
    ff = build_part("feed_forward", ff_spec, _rt(dtype))
    t = {n: rand(*s.shape, seed=i, scale=0.3).to(torch.bfloat16) for i, (n, s) in enumerate(ff.tensor_specs().items())}
    ff.bind(t)
    x = rand(T, W, seed=9, scale=1.5).to(dtype)
    res = torch.zeros(T, W, device=DEV)
    ff.forward(x.to(DEV), res)
    want = PZ.gated_gelu(x.double(), *(t["mlp." + k].double() for k in ("gate", "up", "down")))
    assert max_rel_err(res, want) <= PART_TOL[dtype]
    norm = lambda n: PartSpec("rmsnorm", {"size": W, "eps": 1e-3, "names": {"weight": n}})
    spec = LayerSpec(block="parallel", mixer=PartSpec("general_delta", {"hidden_size": W, "num_heads": 2, "head_dim": 16, "eps": 1e-3, "rank": 8}),
                     feed_forward=ff_spec, norms={"mixer": norm("norm1"), "feed_forward": norm("norm2")}, weight_prefix="")
    block = build_block(spec, _rt(dtype))
    bt, _ = _bf16_weights(block, 0.25, seed=3)
    block.bind(bt)
    storage = CacheStorage([block.mixer.cache_spec()], [None], 8, 8, 1, dtype, torch.device(DEV))
    storage.manager.admit("r")
    batch = build_step_batch([StepEntry("r", [0] * T, [])], storage.manager, torch.device(DEV), 8)
    r0 = rand(T, W, seed=12)
    res = r0.clone().to(DEV)
    block.forward(res, batch, storage.layers[0])
    d = {k: v.double() for k, v in bt.items()}
    mw = {k.split("mix.", 1)[1]: v for k, v in d.items() if k.startswith("mix.")}
    want = r0.double() + PZ.general_delta_mixer(PZ.rms_norm(r0.double(), d["norm1"], 1e-3), mw, {"heads": 2, "dim": 16}, 1e-3) \
        + PZ.gated_gelu(PZ.rms_norm(r0.double(), d["norm2"], 1e-3), d["mlp.gate"], d["mlp.up"], d["mlp.down"])
    assert max_rel_err(res, want) <= PART_TOL[dtype]


def test_embedding_scale():
    from forge_b200 import kernels
    table = rand(20, 12).to(torch.bfloat16).to(DEV)
    ids = torch.tensor([3, 19, 0], dtype=torch.int32, device=DEV)
    assert torch.equal(kernels.embedding(ids, table, scale=0.375).cpu(), table.float().cpu()[[3, 19, 0]] * 0.375)


# ----------------------------------------------------------------------------------------------- whole models

@pytest.fixture(scope="module", params=["P", "Q", "R"])
def zat(request, tmp_path_factory):
    name = request.param
    d = make_zat_dir(tmp_path_factory, name)
    plain = PZ.PlainZatupel(d)
    reqs = {f"r{i}": random_tokens(n, ZAT[name]["vocab"], seed=10 * i + ord(name)) for i, n in enumerate(LENGTHS[name])}
    want = {rid: plain.logits(toks).float() for rid, toks in reqs.items()}
    return name, d, plain, reqs, want


def make_runner(model_dir, dtype, cache_tokens, page_size=8, **kw):
    from forge_b200.engine import ModelRunner
    return ModelRunner(model_dir, dtype=dtype, page_size=page_size, cache_tokens=cache_tokens, max_requests=4, **kw)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("schedule", ["whole", "last_one_by_one", "changing_portions", "mixed"])
def test_schedules_equal_plain(zat, dtype, schedule):
    name, d, plain, reqs, want = zat
    steps = getattr(schedules, schedule)(reqs)
    # exactly as many pages as the schedule's peak needs (were no window to give any back): freed pages and slots are
    # taken again at once
    runner = make_runner(d, dtype, schedules.peak_tokens(reqs, steps, round_to=8))
    got = run_schedule(runner, reqs, steps)
    assert first_bad(got, want, TOL[dtype]) is None, first_bad(got, want, TOL[dtype])
    assert runner.manager.num_free_pages() == {g: runner.num_pages for g in runner.manager.groups}


@pytest.mark.parametrize("dtype", DTYPES)
def test_page_size_and_graphs_do_not_matter(zat, dtype):
    name, d, plain, reqs, want = zat
    small = {k: reqs[k] for k in list(reqs)[:3]}
    for ps, graphs in ((16, True), (64, True), (8, False)):
        steps = schedules.mixed(small, max_live=2)
        runner = make_runner(d, dtype, schedules.peak_tokens(small, steps, round_to=ps), page_size=ps, cuda_graphs=graphs)
        got = run_schedule(runner, small, steps)
        msg = first_bad(got, {k: want[k] for k in small}, TOL[dtype])
        assert msg is None, f"page size {ps}: {msg}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_and_first_tokens(zat, dtype):
    """Two tokens, one, then hundreds one by one: windows pass over decoded tokens, pages go back, state runs long."""
    name, d, plain, reqs, want = zat
    n = {"P": 230, "Q": 260, "R": 170}[name]
    toks = random_tokens(n, ZAT[name]["vocab"], seed=77)
    ref = plain.logits(toks).float()
    runner = make_runner(d, dtype, -(-n // 8) * 8)
    steps = [([("x", 0, 2)], [])] + [([("x", p, 1)], []) for p in range(2, n)]
    got = run_schedule(runner, {"x": toks}, steps)
    msg = first_bad(got, {"x": ref}, TOL[dtype])
    assert msg is None, msg


def test_fp32_logits_do_not_depend_on_the_cut(zat):
    """In 32-bit every sum is taken in an order that the position alone decides: the four schedules give the same bits."""
    name, d, plain, reqs, want = zat
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
def test_generation_through_the_scheduler(zat, dtype):
    """Greedy generation through forge.Model and through RequestScheduler with more requests than slots and few pages."""
    import forge_b200 as forge
    name, d, plain, reqs, want = zat
    model = forge.Model(d, dtype=dtype, block_size=8, max_num_seqs=2, cache_tokens=512, max_tokens_per_step=48)
    prompt = reqs["r1"][:37]
    out = model.generate(prompt, max_new_tokens=12, do_sample=False)
    assert out["num_generated_tokens"] == 12 and out["finish_reason"] == "length"
    logits_fn = lambda ids: plain.logits(ids).float()
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


def test_trace_replay_as_a_subprocess(zat, tmp_path):
    name, d, plain, reqs, want = zat
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
    V = ZAT[name]["vocab"]
    for n, rows in asked.items():
        got = torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(len(rows), V))
        ref = torch.stack([want[rid][pos] for rid, pos in rows])
        assert max_rel_err(got, ref) <= TOL["float32"], n
    assert sorted(os.listdir(out)) == sorted(f"{n}.f32" for n in asked)
