"""Redasun through the framework against the plain implementation (plain_redasun.py): configuration and names, cache groups, each
mechanism alone (the plain functions' own properties, the kernels by themselves, models of one kind of layer), and the engine's step
function under every way of cutting the work.  The ``gpu`` tests run the kernels; the others need no device."""
from __future__ import annotations

import json
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_redasun
import trace_tools
from tinyllama_inference_engine_b200 import EngineConfig
from tinyllama_inference_engine_b200.cache import CacheManager
from tinyllama_inference_engine_b200.config import architecture_for, load_model_config
from tinyllama_inference_engine_b200.engine.batch import StepEntry
from tinyllama_inference_engine_b200.engine.runner import ModelRunner
from tinyllama_inference_engine_b200.errors import ConfigError
from tinyllama_inference_engine_b200.models import cache_needs, expected_tensors
from tinyllama_inference_engine_b200.models.redasun_config import RedasunConfig
from tinyllama_inference_engine_b200.weights import SafetensorsFile, write_random_model, write_safetensors


def _dense(ff):
    return None if ff is None else {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, groups=None, shared=None, scale=1.5):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router, "shared": None if shared is None else {"ff": shared}}


def _layer(heads, kv_heads, dim, vdim, mlp, rot=None, base=10000.0, diff=0.3, scale=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else 2.0 * dim ** -0.5, "diff": diff}
    if rot is not None:
        mixer["rot"] = {"base": base, "dims": rot}
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def _config(width, vocab, layers, loop=None, eps=1e-5, embed_scale=None):
    data = {"architecture": "Redasun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": width ** 0.5 if embed_scale is None else embed_scale},
            "layers": layers}
    if loop:
        data["loop"] = dict(zip(("start", "stop", "times"), loop))
    return data


# Sizes that agree nowhere: grouped and ungrouped heads, one head, key and value widths equal and not, multiples of 16 (the tensor-core
# kernel's sizes) and not, rotations of the whole vector, of a part and of nothing, layers with a dense feed-forward, with experts (in
# groups of which some are dropped, in one group, one expert per token, without a shared expert) and with none, a repeated run in the
# middle, over the whole model, once, and none.
CONFIGS = {
    "all": (_config(64, 97, [_layer(4, 2, 16, 32, _dense(48), rot=8), _layer(2, 1, 32, 16, _moe(8, 3, 24, groups=(4, 2), shared=40), rot=32, base=500.0),
                             _layer(3, 3, 16, 16, None, rot=4, diff=0.6), _layer(4, 1, 16, 48, _moe(6, 2, 16, shared=None), rot=16)], loop=(1, 3, 3)), 3),
    "whole_loop": (_config(48, 61, [_layer(2, 2, 24, 8, _moe(4, 1, 32, groups=(2, 1), shared=16, scale=1.0)), _layer(6, 2, 8, 16, _dense(40), rot=8, diff=0.0)], loop=(0, 2, 2),
                           embed_scale=5.0, eps=1e-6), 5),
    "plain_order": (_config(40, 53, [_layer(1, 1, 40, 40, _dense(24), rot=20), _layer(5, 1, 8, 8, _moe(9, 4, 8, groups=(3, 2), shared=8), rot=2, base=50.0)]), 9),
    "one_pass": (_config(32, 50, [_layer(4, 4, 16, 16, _dense(16), rot=16), _layer(2, 2, 16, 32, _moe(4, 2, 16, groups=(4, 3), shared=24), rot=6)], loop=(1, 2, 1)), 4),
    # nothing a multiple of 8: the width, the vocabulary, the feed-forwards, the heads' widths
    "odd": (_config(44, 37, [_layer(3, 1, 12, 10, _moe(6, 2, 10, groups=(3, 2), shared=6), rot=6), _layer(2, 2, 10, 6, _dense(50), rot=10)], loop=(0, 1, 2)), 8),
}
LENGTHS = {"all": [1, 9, 70, 150, 33, 64, 17], "whole_loop": [3, 40, 100, 64, 7], "plain_order": [2, 130, 65, 16, 200], "one_pass": [90, 5, 48, 17], "odd": [70, 3, 33, 18]}
TOLERANCE = {"float32": 3e-5, "bfloat16": 2.5e-2}     # 32-bit: of a row's largest difference; bfloat16: of its root mean square over the vocabulary
RMS = {"float32": False, "bfloat16": True}


def load_plain(folder, dtype=torch.float32):
    config = json.loads((folder / "config.json").read_text())
    file = SafetensorsFile(folder / "model.safetensors")
    tensors = {name: file.tensor(name).clone().to(dtype) for name in file.names()}
    file.close()
    return config, tensors


def _logits(config, tensors, tokens):
    return plain_redasun.forward(config, tensors, tokens)[0]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("redasun")
    return {key: write_random_model(base / key, config, seed) for key, (config, seed) in CONFIGS.items()}


@pytest.fixture(scope="module")
def cases(folders):
    out = {}
    for key, folder in folders.items():
        config, tensors = load_plain(folder)
        requests = trace_tools.make_requests(config["vocab"], LENGTHS[key], seed=21)
        full = {rid: _logits(config, tensors, tokens) for rid, tokens in requests.items()}
        out[key] = (folder, requests, full, max(float(v.abs().max()) for v in full.values()))
    return out


def _runner(folder, dtype, max_tokens=1024, page_size=16, requests=4):
    return ModelRunner(folder, EngineConfig(dtype=dtype, page_size=page_size, max_cache_tokens=max_tokens, max_requests=requests, max_batch_tokens=1024,
                                            device="cuda:0", poison_freed_pages=True, use_cuda_graphs=False))


def _schedules(requests, seed=3, page_size=16):
    mixed, peak = trace_tools.mixed(requests, seed=seed, page_size=page_size)
    return {"whole": (trace_tools.whole(requests), 1024), "decode": (trace_tools.tail_decode(requests), 1024), "portions": (trace_tools.portions(requests), 1024),
            "mixed": (mixed, peak)}   # a pool of exactly the peak: pages are used again


# --- configuration, registry, names, cache groups -----------------------------------------------------------------------------------
def test_configuration_round_trip_registry_and_names(folders):
    architecture, config = load_model_config(folders["all"])
    assert architecture.name == "Redasun" and isinstance(config, RedasunConfig)
    assert RedasunConfig.from_dict(config.to_dict()) == config
    assert config.layers[2]["mlp"] is None and config.loop == {"start": 1, "stop": 3, "times": 3}
    assert config.layers[3]["mlp"]["router"]["groups"] == {"count": 1, "keep": 1} and config.layers[3]["mlp"]["shared"] is None
    spec = architecture.build_spec(config)
    names = {t.name: tuple(t.shape) for t in expected_tensors(spec)}
    assert names["embed"] == (97, 64) and names["loop.in"] == (64, 128) and names["final.norm"] == (64,) and "head" not in names
    assert names["l0.mix.q"] == (128, 64) and names["l0.mix.k"] == (64, 64) and names["l0.mix.v"] == (64, 64) and names["l0.mix.o"] == (64, 128)
    assert names["l0.mix.q.norm"] == (16,) and names["l0.mix.lk2"] == (16,) and names["l0.norm1b"] == (64,) and names["l0.norm2b"] == (64,)
    assert names["l0.mlp.gate"] == (48, 64) and names["l0.mlp.down"] == (64, 48)
    assert names["l1.mlp.e7.up"] == (24, 64) and names["l1.mlp.e0.down"] == (64, 24) and names["l1.mlp.router"] == (8, 64) and names["l1.mlp.correction"] == (8,)
    assert names["l1.mlp.shared.gate"] == (40, 64) and "l3.mlp.shared.gate" not in names and "l2.norm2" not in names and "l2.mlp.gate" not in names
    runs = [(spec.layers[e.layer].prefix, e.cache) for e in spec.order]
    assert [p for p, _ in runs] == ["l0", "loop", "l1", "l2", "loop", "l1", "l2", "loop", "l1", "l2", "l3"] and len({c for _, c in runs}) == len(runs)
    assert plain_redasun.runs_of(CONFIGS["all"][0]) == [(0, False), (1, True), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    # a pass of a run that repeats once still starts with the input mix
    spec = architecture.build_spec(RedasunConfig.from_dict(CONFIGS["one_pass"][0]))
    assert [spec.layers[e.layer].prefix for e in spec.order] == ["l0", "loop", "l1"]


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="lstm"), "type"),
    (lambda c: c["layers"][0].update(mlp={"kind": "routed", "ff": 8}), "kind"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].update(diff=1.0), "diff"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "experts"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=3), "experts"),
    (lambda c: c.update(loop={"start": 2, "stop": 2, "times": 2}), "loop"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_configuration_refuses_what_the_design_lacks(change, message):
    data = json.loads(json.dumps(CONFIGS["all"][0]))
    change(data)
    with pytest.raises(ConfigError, match=message):
        RedasunConfig.from_dict(data)


def test_cache_groups():
    """Runs of equal key and value planes share a group; a layer's key plane holds two vectors per key/value head."""
    architecture = architecture_for(CONFIGS["all"][0])
    needs = cache_needs(architecture.build_spec(architecture.config_class.from_dict(CONFIGS["all"][0])))
    manager = CacheManager(needs, page_size=16, num_pages=40, max_requests=2, max_positions=4096)
    groups = sorted((g.need.page_planes(), len(g.streams)) for g in manager.page_groups)
    assert groups == [(((2, 16), (1, 48)), 1), (((2, 32), (1, 16)), 3), (((4, 16), (2, 32)), 1), (((6, 16), (3, 16)), 3)]


# --- the plain implementation's own mechanisms --------------------------------------------------------------------------------------
def _random_weights(shapes, seed):
    g = torch.Generator().manual_seed(seed)
    return {name: torch.randn(shape, generator=g, dtype=torch.float64) * (shape[-1] ** -0.5 if len(shape) > 1 else 1.0) for name, shape in shapes.items()}


def test_plain_maps_cancel_and_rotation_is_relative():
    sizes = {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 6, "scale": 0.7, "diff": 0.25, "rot": {"base": 100.0, "dims": 4}}
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(9, n, d, generator=g, dtype=torch.float64) for n, d in ((4, 8), (2, 8), (1, 6)))
    ones = torch.ones(8, dtype=torch.float64)
    positions = torch.arange(9)
    out = plain_redasun.two_map_heads(q, k, v, positions, sizes, 1e-6, 0.4, ones, ones)
    # every head's output has a root mean square of 1 - diff, whatever lambda is
    assert torch.allclose((out * out).mean(-1).sqrt(), torch.full((9, 2), 0.75, dtype=torch.float64), atol=1e-5)
    # equal maps: with lambda = 1 nothing but rounding noise would be left, so lambda decides
    same_q = q.clone()
    same_q[:, 1::2] = same_q[:, 0::2]
    same_k = k.clone()
    same_k[:, 1::2] = same_k[:, 0::2]
    half = plain_redasun.two_map_heads(same_q, same_k, v, positions, sizes, 1e-6, 0.5, ones, ones)
    none = plain_redasun.two_map_heads(same_q, same_k, v, positions, sizes, 1e-6, 0.0, ones, ones)
    assert torch.allclose(half, none, atol=1e-5)       # (1 - 0.5) a, normalised, is a normalised (but for eps)
    # the first token sees itself alone: its maps are its value, whatever q and k are
    first = plain_redasun.two_map_heads(q, k, v, positions, sizes, 1e-6, 0.4, ones, ones)[0, 0]
    assert torch.allclose(first, plain_redasun.rms(v[0, 0] * 0.6, 1e-6) * 0.75, atol=1e-9)
    x = torch.randn(5, 3, 8, generator=g, dtype=torch.float64)
    turned = plain_redasun.rotate_front(x, torch.arange(5), 4, 100.0)
    assert torch.equal(turned[..., 4:], x[..., 4:]) and torch.equal(turned[0], x[0]) and torch.allclose((turned * turned).sum(-1), (x * x).sum(-1))
    later = plain_redasun.rotate_front(x, torch.arange(5) + 7, 4, 100.0)
    assert torch.allclose((turned[3, 0] * turned[1, 1]).sum(), (later[3, 0] * later[1, 1]).sum())     # a score depends on the distance only
    assert torch.allclose(turned[2, 0, 0], x[2, 0, 0] * np.cos(2.0) - x[2, 0, 2] * np.sin(2.0))          # column 0 turns with column 2 = dims / 2


def test_plain_router_drops_groups_and_weighs_without_the_correction():
    router = {"experts": 6, "top": 2, "scale": 3.0, "groups": {"count": 3, "keep": 1}}
    # one token whose router logits are the rows of an identity-like matrix: z = the token's first six numbers
    tensors = {"m.router": torch.eye(6, 8), "m.correction": torch.tensor([0.0, 0.0, 0.0, 0.0, -2.0, -2.0])}
    h = torch.tensor([[4.0, -9.0, 1.0, 1.5, 3.0, 3.5, 0.0, 0.0]])
    chosen, weights = plain_redasun.route(h, tensors, "m", router)
    # expert 0 has the largest score, but its group's two best (0.98 + 0.0) lose to group 1's (0.73 + 0.82); group 2 is pushed below by its correction
    assert chosen == [[3, 2]]
    s = torch.sigmoid(torch.tensor([1.5, 1.0]))
    assert np.allclose(weights[0], (s / s.sum() * 3.0).tolist())
    router["groups"] = {"count": 3, "keep": 3}
    assert plain_redasun.route(h, tensors, "m", router)[0] == [[0, 3]]
    # every choice score below zero: the kept group's experts (about -4) still beat the dropped ones, which count as minus infinity and not as 0
    tensors["m.correction"] = torch.full((6,), -5.0)
    router["groups"] = {"count": 3, "keep": 1}
    chosen, weights = plain_redasun.route(h, tensors, "m", router)
    assert chosen == [[5, 4]] and np.allclose(sum(weights[0]), 3.0)


def test_plain_layer_norm_and_order_of_runs():
    x = torch.randn(3, 10, dtype=torch.float64)
    w = torch.randn(10, dtype=torch.float64)
    want = torch.nn.functional.layer_norm(x, (10,), w, None, 1e-5)
    assert torch.allclose(plain_redasun.layer_norm(x, w, 1e-5), want)
    assert plain_redasun.runs_of({"layers": [0, 1, 2]}) == [(0, False), (1, False), (2, False)]
    assert plain_redasun.runs_of({"layers": [0, 1, 2], "loop": {"start": 0, "stop": 2, "times": 2}}) == [(0, True), (1, False), (0, True), (1, False), (2, False)]


# --- kernels by themselves ------------------------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype,atol", [(torch.float32, 3e-6), (torch.bfloat16, 1.2e-2)])
@pytest.mark.parametrize("centred", [True, False])
@pytest.mark.parametrize("width", [44, 256, 1000])
def test_branch_norm_kernel(dtype, atol, centred, width):
    from tinyllama_inference_engine_b200 import ops

    g = torch.Generator().manual_seed(width)
    stream = torch.randn(9, width, generator=g) * 3.0 + 1.0
    y = (torch.randn(9, width, generator=g) * 2.0 - 0.5).to(dtype)
    post, following = 1 + 0.1 * torch.randn(width, generator=g), 1 + 0.1 * torch.randn(width, generator=g)
    norm = plain_redasun.layer_norm if centred else (lambda x, w, eps: plain_redasun.rms(x, eps) * w)
    want_stream = stream.double() + norm(y.double(), post.double(), 1e-5)
    want_out = norm(want_stream, following.double(), 1e-5)
    residual = stream.cuda()
    out = torch.zeros(9, width, dtype=dtype, device="cuda")
    ops.branch_norm(residual, y.cuda(), post.cuda(), following.cuda(), out, 1e-5, centred)
    assert float((residual.cpu().double() - want_stream).abs().max()) <= 3e-6 * float(want_stream.abs().max())
    assert float((out.cpu().double() - want_out).abs().max()) <= atol * float(want_out.abs().max())
    rows = torch.tensor([7, 2, 2], dtype=torch.int32).cuda()
    some = torch.zeros(3, width, dtype=dtype, device="cuda")
    ops.branch_norm(residual, None, None, following.cuda(), some, 1e-5, centred, rows)
    assert torch.equal(some.cpu(), out.cpu()[[7, 2, 2]])
    only_add = stream.cuda()
    ops.branch_norm(only_add, y.cuda(), post.cuda(), None, None, 1e-5, centred)
    assert torch.equal(only_add, residual)


def _attention_case(dtype, heads, kv, dim, vdim, lens, firsts, page_size, seed):
    """Whole requests' q, k, v rows; the rows of the first step (positions below ``firsts``) and of the second; pages in a scrambled order."""
    from tinyllama_inference_engine_b200.parts.base import CacheNeed, LayerCache

    g = torch.Generator().manual_seed(seed)
    totals = [f + n for n, f in zip(lens, firsts)]
    width = max(-(-t // page_size) for t in totals)
    count = sum(-(-t // page_size) for t in totals) + 3
    order = torch.randperm(count, generator=g).tolist()
    table = torch.full((len(lens), width), -1, dtype=torch.int32)
    for r, t in enumerate(totals):
        for p in range(-(-t // page_size)):
            table[r, p] = order.pop()
    columns = 2 * heads * dim + 2 * kv * dim + kv * vdim
    columns += -columns % 8
    rows = [torch.randn(t, columns, generator=g).to(dtype) for t in totals]
    planes = (torch.full((count, 2 * kv, page_size, dim), float("nan")).to(dtype).cuda(), torch.full((count, kv, page_size, vdim), float("nan")).to(dtype).cuda())
    cache = LayerCache(CacheNeed("pages"), True, None, table.cuda(), page_size, None, planes)
    return rows, cache


def _step_of(rows, cache, pieces):
    """The context of a step that brings request r's rows [a, a + n) for (r, a, n) in ``pieces``."""
    index = [(r, a + i) for r, a, n in pieces for i in range(n)]
    step_rows = torch.stack([rows[r][p] for r, p in index]).cuda().contiguous()
    positions = torch.tensor([p for _, p in index], dtype=torch.int32).cuda()
    token_seq = torch.tensor([j for j, (_, _, n) in enumerate(pieces) for _ in range(n)], dtype=torch.int32).cuda()
    starts = torch.tensor(np.concatenate([[0], np.cumsum([n for _, _, n in pieces])]), dtype=torch.int32).cuda()
    sub = type(cache)(cache.need, True, None, cache.block_table[[r for r, _, _ in pieces]].contiguous(), cache.page_size, None, cache.plane_pages)
    batch = SimpleNamespace(max_q_len=max(n for _, _, n in pieces), num_seqs=len(pieces), max_seq_len=max(a + n for _, a, n in pieces), seq_starts=starts,
                            first_positions=torch.tensor([a for _, a, _ in pieces], dtype=torch.int32).cuda(), num_tokens=len(index))
    return step_rows, positions, token_seq, sub, batch, index


ATTENTION_SHAPES = [(4, 2, 16, 32, 8), (2, 1, 32, 16, 32), (3, 3, 16, 16, 0), (6, 1, 64, 64, 20), (1, 1, 40, 24, 10), (5, 5, 10, 6, 4), (8, 2, 128, 128, 64), (20, 1, 16, 16, 16)]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,atol", [(torch.float32, 2e-5), (torch.bfloat16, 6e-2)])    # bfloat16: q and the cached k, v are rounded, and dividing the
@pytest.mark.parametrize("heads,kv,dim,vdim,rot", ATTENTION_SHAPES)                         # difference of two maps by its root mean square amplifies that
@pytest.mark.parametrize("with_batch,long_tail", [(False, False), (True, False), (True, True)])
def test_differential_attention_kernels(dtype, atol, heads, kv, dim, vdim, rot, with_batch, long_tail):
    """Norm, rotation, cache write and the two maps against the plain function: every request in two steps, so that the second reads
    what the first cached through a scrambled block table; a portion from position 0, a decoded token and a portion that starts
    inside a page.  With the step's context the kernels are chosen as the engine chooses them (tensor cores for portions, a row's
    keys cut into runs for steps of few rows); without it the general kernel runs alone.  The last rows of every request form a third
    step of few rows per entry (the kernel whose rows are a token's heads), over a few tiles of keys or over many."""
    from tinyllama_inference_engine_b200 import ops

    lens, firsts, page_size = ([37, 1, 18], [30, 52, 0], 16) if not long_tail else ([5, 150, 9], [330, 0, 61], 16)
    rows, cache = _attention_case(dtype, heads, kv, dim, vdim, lens, firsts, page_size, seed=heads * 100 + dim)
    g = torch.Generator().manual_seed(7)
    q_weight, k_weight = 1 + 0.2 * torch.randn(dim, generator=g), 1 + 0.2 * torch.randn(dim, generator=g)
    sizes = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": 1.5 * dim ** -0.5, "diff": 0.3, "rot": {"base": 300.0, "dims": rot}}
    lam, eps = 0.45, 1e-5
    inv_freq = torch.tensor([300.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32).cuda()
    k_offset, v_offset = 2 * heads * dim, 2 * heads * dim + 2 * kv * dim
    want = []
    for r in rows:
        x = r.double()
        total = x.shape[0]
        q, k, v = x[:, :k_offset].view(total, 2 * heads, dim), x[:, k_offset:v_offset].view(total, 2 * kv, dim), x[:, v_offset : v_offset + kv * vdim].view(total, kv, vdim)
        want.append(plain_redasun.two_map_heads(q, k, v, torch.arange(total), sizes, eps, lam, q_weight.double(), k_weight.double()).reshape(total, heads * vdim))
    got = [torch.zeros_like(w) for w in want]
    tails = [min(n, 3 + r) for r, n in enumerate(lens)]   # every request's last rows come as a step of few rows of their own
    for pieces in ([(r, 0, f) for r, f in enumerate(firsts) if f > 0], [(r, f, n - t) for r, (n, f, t) in enumerate(zip(lens, firsts, tails)) if n > t],
                   [(r, f + n - t, t) for r, (n, f, t) in enumerate(zip(lens, firsts, tails))]):
        step_rows, positions, token_seq, sub, batch, index = _step_of(rows, cache, pieces)
        ops.diff_store(step_rows, k_offset, v_offset, q_weight.cuda(), k_weight.cuda(), eps, inv_freq, rot, positions, token_seq, sub, heads, kv, dim, vdim)
        out = torch.zeros(len(index), heads * vdim, dtype=dtype, device="cuda")
        ops.diff_attention(step_rows, positions, token_seq, sub, out, heads, kv, dim, vdim, sizes["scale"], lam, eps, 0.7, batch=batch if with_batch else None)
        for (r, p), row in zip(index, out.cpu().double()):
            got[r][p] = row
    for r in range(len(rows)):
        assert float((got[r] - want[r]).abs().max()) <= atol * (2.5 if long_tail else 1.0), r    # hundreds of keys: longer 32-bit sums under the same division


@pytest.mark.gpu
@pytest.mark.parametrize("tokens", [50, 1300])    # a CTA per token; four tokens per CTA (a step of many rows), the last CTA short of rows
@pytest.mark.parametrize("experts,groups,keep,top,width", [(8, 4, 2, 3, 64), (6, 1, 1, 2, 44), (9, 3, 2, 4, 40), (4, 4, 3, 2, 32), (64, 8, 4, 8, 128), (5, 5, 1, 1, 24), (12, 2, 1, 6, 48),
                                                           (10, 5, 2, 3, 42), (7, 1, 1, 7, 17)])    # rows that are no multiple of four numbers: the general form
def test_router_kernel(tokens, experts, groups, keep, top, width):
    """The chosen experts and their weights against the plain router; corrections large enough to push choice scores below zero."""
    from tinyllama_inference_engine_b200 import ops

    g = torch.Generator().manual_seed(experts * 7 + width)
    x = torch.randn(tokens, width, generator=g)
    tensors = {"m.router": torch.randn(experts, width, generator=g) * 2.0 * width ** -0.5, "m.correction": torch.randn(experts, generator=g) - 0.8}
    router = {"experts": experts, "top": top, "scale": 2.5, "groups": {"count": groups, "keep": keep}}
    chosen, weights = plain_redasun.route(x, tensors, "m", router)
    ids = torch.zeros(tokens, top, dtype=torch.int32, device="cuda")
    got = torch.zeros(tokens, top, device="cuda")
    ops.moe_route(x.cuda(), tensors["m.router"].cuda(), tensors["m.correction"].cuda(), ids, got, groups, keep, 2.5)
    wrong = [t for t in range(tokens) if ids[t].cpu().tolist() != chosen[t]]
    # another order of the sum may turn a choice only where two choice scores all but tie
    for t in wrong:
        z = torch.sigmoid(tensors["m.router"].double() @ x[t].double()) + tensors["m.correction"].double()
        gaps = (z[:, None] - z[None, :]).abs() + torch.eye(experts, dtype=torch.float64)
        assert float(gaps.min()) < 1e-5, t
    right = [t for t in range(tokens) if t not in wrong]
    assert len(right) >= tokens - 2
    assert torch.allclose(got.cpu()[right], torch.tensor(weights)[right], atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,atol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("tokens,experts,top,width,ff,shared", [(5, 6, 2, 44, 10, True), (70, 8, 3, 64, 24, True), (300, 4, 1, 32, 16, False), (130, 16, 4, 128, 48, True), (1, 3, 3, 24, 8, False),
                                                                (300, 4, 1, 64, 72, False), (700, 6, 3, 136, 200, True)])   # enough rows per expert for tiles of 128 rows on tcgen05
def test_expert_kernels(dtype, atol, tokens, experts, top, width, ff, shared):
    """The chosen experts' gated feed-forwards, weighted and summed with the shared branch: steps of few rows read the experts' rows
    directly, bfloat16 prompt portions sort by expert and use the tensor cores."""
    from tinyllama_inference_engine_b200 import ops

    g = torch.Generator().manual_seed(tokens + experts)
    x = torch.randn(tokens, width, generator=g).to(dtype)
    gate_up = (torch.randn(experts, 2 * ff, width, generator=g) * width ** -0.5).to(dtype)
    down = (torch.randn(experts, width, ff, generator=g) * ff ** -0.5).to(dtype)
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(tokens)]).to(torch.int32)
    weights = torch.rand(tokens, top, generator=g) + 0.1
    branch = torch.randn(tokens, width, generator=g).to(dtype) if shared else None
    want = torch.zeros(tokens, width, dtype=torch.float64) if branch is None else branch.double().clone()
    for t in range(tokens):
        for k in range(top):
            e = int(ids[t, k])
            z = gate_up[e].double() @ x[t].double()
            want[t] += float(weights[t, k]) * (down[e].double() @ (z[:ff] * torch.sigmoid(z[:ff]) * z[ff:]))
    got = torch.zeros(tokens, width, dtype=dtype, device="cuda")
    ops.moe_experts(x.cuda(), gate_up.cuda(), down.cuda(), ids.cuda(), weights.cuda(), None if branch is None else branch.cuda(), got, "silu")
    assert float((got.cpu().double() - want).abs().max()) <= atol * max(1.0, float(want.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("activation", ["silu", "gelu_tanh"])
def test_expert_kernels_with_idle_and_crowded_experts(activation):
    """Experts that no token chose, one that most chose (several row tiles) and one with a single row, at a width and an expert size that are
    multiples of 8 only; a token's result does not depend on what else is in the step."""
    from tinyllama_inference_engine_b200 import ops

    tokens, experts, top, width, ff = 900, 7, 2, 72, 88
    g = torch.Generator().manual_seed(11)
    x = torch.randn(tokens, width, generator=g).bfloat16()
    gate_up = (torch.randn(experts, 2 * ff, width, generator=g) * width ** -0.5).bfloat16()
    down = (torch.randn(experts, width, ff, generator=g) * ff ** -0.5).bfloat16()
    ids = torch.empty(tokens, top, dtype=torch.int32)
    ids[:, 0] = 3                                                    # every token: the crowded expert
    ids[:, 1] = torch.where(torch.arange(tokens) % 3 == 0, 5, 1)     # experts 0, 2, 4 and 6 stay idle
    ids[17, 1] = 6                                                   # one row
    weights = torch.rand(tokens, top, generator=g) + 0.1
    z = torch.einsum("efw,tw->tef", gate_up.double(), x.double())
    gate, up = z[:, :, :ff], z[:, :, ff:]
    act = (gate * torch.sigmoid(gate) if activation == "silu" else plain_redasun.gelu_tanh(gate)) * up
    y = torch.einsum("ewf,tef->tew", down.double(), act)
    want = sum(weights[:, k, None].double() * y[torch.arange(tokens), ids[:, k].long()] for k in range(top))
    got = torch.zeros(tokens, width, dtype=torch.bfloat16, device="cuda")
    args = (gate_up.cuda(), down.cuda())
    ops.moe_experts(x.cuda(), *args, ids.cuda(), weights.cuda(), None, got, activation)
    assert int(ops.error_flag(got.device)) == 0
    assert float((got.cpu().double() - want).abs().max()) <= 2e-2 * max(1.0, float(want.abs().max()))
    some = torch.tensor([17, 0, 899, 450, 3])
    alone = torch.zeros(len(some), width, dtype=torch.bfloat16, device="cuda")
    ops.moe_experts(x[some].cuda(), *args, ids[some].cuda(), weights[some].cuda(), None, alone, activation)
    assert float((alone.float().cpu() - got.float().cpu()[some]).abs().max()) <= 2e-2 * max(1.0, float(want.abs().max()))


@pytest.mark.gpu
def test_gelu_gate_of_few_rows_and_of_many():
    """gelu(gate) * up in the small-step product's epilogue (one kernel, up to 16 rows) gives what the product and the row-wise kernel give."""
    from tinyllama_inference_engine_b200 import ops

    g = torch.Generator().manual_seed(5)
    weight = (torch.randn(2 * 72, 64, generator=g) * 0.3).bfloat16().cuda()
    for rows in (1, 7, 16, 40):
        x = torch.randn(rows, 64, generator=g).bfloat16().cuda()
        got = torch.zeros(rows, 72, dtype=torch.bfloat16, device="cuda")
        before = ops.launch_count
        ops.linear_gated(x, weight, got, activation="gelu_tanh")
        assert rows > 16 or ops.launch_count - before == 1
        reference = x.float().cpu() @ weight.float().cpu().T
        plain = plain_redasun.gelu_tanh(reference[:, :72]) * reference[:, 72:]
        assert torch.allclose(got.float().cpu(), plain, atol=3e-2, rtol=3e-2)
    x32, w32 = torch.randn(9, 64, generator=g).cuda(), weight.float()
    gate_up, out = torch.zeros(9, 144, device="cuda"), torch.zeros(9, 72, device="cuda")
    ops.linear(x32, w32, gate_up)
    ops.gate_mul(gate_up, out, "gelu_tanh")
    assert torch.allclose(out.cpu(), plain_redasun.gelu_tanh(gate_up[:, :72].cpu()) * gate_up[:, 72:].cpu(), atol=1e-6, rtol=1e-5)


# --- the engine on the GPU under every way of cutting the work ---------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", list(CONFIGS))
def test_engine_matches_plain_under_every_schedule(cases, key, dtype):
    """Whole prompts, a tail decoded token by token, portions down to two tokens, and four live requests mixed in a pool that makes
    pages come round again (freed pages are poisoned with NaN)."""
    folder, requests, full, scale = cases[key]
    for name, (steps, pool) in _schedules(requests).items():
        runner = _runner(folder, dtype, max_tokens=pool)
        trace_tools.run_and_compare(runner, steps, full, atol=TOLERANCE[dtype] * scale, over_vocabulary=RMS[dtype])
        runner.cache.check()
        assert not runner.cache.records, name
        if name == "mixed":
            assert all(g.pool.reuses > 0 for g in runner.cache.page_groups)


@pytest.mark.gpu
def test_layer_outputs_match_the_plain_trace(cases):
    folder, requests, full, scale = cases["all"]
    config, tensors = load_plain(folder)
    tokens = requests["r4"]
    want = plain_redasun.forward(config, tensors, tokens)[1]
    trace = {}
    _runner(folder, "float32").step([StepEntry("a", tokens, [0])], trace=trace)
    assert len(trace) == len(want) == 8          # the input mix that starts a pass is no layer of its own
    for index, layer in enumerate(want):
        assert float((trace[f"layer{index}.output"].cpu() - layer).abs().max()) <= 3e-5 * float(layer.abs().max()), index


def _sharpened(folder, name, edit, config_edit=None):
    """A copy of a model folder with some tensors (and constants) changed, so that one mechanism decides the logits."""
    target = folder.parent / f"{folder.name}_{name}"
    target.mkdir(exist_ok=True)
    config = json.loads((folder / "config.json").read_text())
    if config_edit:
        config_edit(config)
    (target / "config.json").write_text(json.dumps(config))
    _, tensors = load_plain(folder, torch.bfloat16)
    edit(tensors)
    write_safetensors(target / "model.safetensors", tensors)
    return target


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_keys_and_first_tokens_decide(folders, dtype):
    """A large score scale lets single keys win a row, hundreds of tokens back and across page borders: a lost key, a key of the wrong
    map or a rotation by the wrong position then moves the logits far beyond the tolerance, in portions, in decoded tokens and in
    mixed batches.  The second map is weighed up (a large lambda), so that leaving it out shows as well."""
    def edit(tensors):
        for name in tensors:
            if name.endswith(".lq1") or name.endswith(".lk1"):
                tensors[name] = torch.full_like(tensors[name], 0.2)

    def sharper(config):
        for layer in config["layers"]:
            layer["mixer"]["scale"] = 2.0

    folder = _sharpened(folders["plain_order"], "sharp", edit, sharper)
    config, tensors = load_plain(folder)
    requests = trace_tools.make_requests(config["vocab"], [400, 70, 33], seed=17)
    full = {rid: _logits(config, tensors, tokens) for rid, tokens in requests.items()}
    scale = max(float(v.abs().max()) for v in full.values())
    early = [(t + 1) % config["vocab"] if 10 <= i < 110 else t for i, t in enumerate(requests["r0"])]       # across page borders, 290 tokens and more back
    assert float((_logits(config, tensors, early)[-1] - full["r0"][-1]).abs().max()) > 50 * TOLERANCE["float32"] * scale
    first = [(requests["r0"][0] + 1) % config["vocab"]] + requests["r0"][1:]
    assert float((_logits(config, tensors, first)[100:] - full["r0"][100:]).abs().max()) > 50 * TOLERANCE["float32"] * scale      # the first token shows hundreds of tokens on
    one_map = {name: (torch.full_like(t, -30.0) if name.endswith(".lq2") else t) for name, t in tensors.items()}
    assert float((_logits(config, one_map, requests["r1"]) - full["r1"]).abs().max()) > 50 * TOLERANCE["float32"] * scale
    for steps in (trace_tools.tail_decode(requests, tail=40), trace_tools.portions(requests), trace_tools.mixed(requests, seed=4, max_portion=90)[0]):
        trace_tools.run_and_compare(_runner(folder, dtype, max_tokens=2048), steps, full, atol=TOLERANCE[dtype] * scale, over_vocabulary=RMS[dtype])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_other_page_sizes(cases, dtype):
    """150 tokens decoded one by one behind a prompt, with pages of 64 and of 32 tokens."""
    folder, requests, full, scale = cases["whole_loop"]
    some = {rid: requests[rid] for rid in ("r2", "r3")}
    more = dict(some, long=trace_tools.make_requests(61, [260], seed=5)["r0"])
    config, tensors = load_plain(folder)
    full = dict(full, long=_logits(config, tensors, more["long"]))
    for page_size in (64, 32):
        trace_tools.run_and_compare(_runner(folder, dtype, max_tokens=2048, page_size=page_size), trace_tools.tail_decode(more, tail=150), full,
                                    atol=TOLERANCE[dtype] * scale, over_vocabulary=RMS[dtype])


@pytest.mark.gpu
def test_rows_do_not_depend_on_the_batch(cases):
    """32-bit rows agree to rounding however the step is cut and whatever else is in the batch."""
    folder, requests, full, scale = cases["all"]
    alone, together = _runner(folder, "float32"), _runner(folder, "float32")
    tokens = requests["r3"]
    whole = alone.step([StepEntry("x", tokens, [len(tokens) - 1])]).cpu()
    together.step([StepEntry("y", requests["r2"][:40], []), StepEntry("x", tokens[:77], [])])
    cut = together.step([StepEntry("x", tokens[77:], [len(tokens) - 78]), StepEntry("y", requests["r2"][40:41], [0])]).cpu()
    assert float((cut[0] - whole[0]).abs().max()) <= 1e-5 * scale


# --- generation through the engine's own entry point -------------------------------------------------------------------------------------
def _plain_greedy(config, tensors, prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(_logits(config, tensors, tokens)[-1].argmax()))
    return tokens[len(prompt):]


@pytest.mark.gpu
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(folders, graphs):
    """Prompts of unequal length through ``Engine.generate``: scheduler, portions under a small token budget, decode sessions (captured as
    graphs or not).  32-bit, so that the plain choice is the engine's."""
    from tinyllama_inference_engine_b200 import Engine, SamplingParams

    folder = folders["all"]
    config, tensors = load_plain(folder)
    rng = np.random.default_rng(31)
    prompts = [[int(t) for t in rng.integers(0, config["vocab"], size=n)] for n in (50, 3, 21, 34, 8)]
    engine = Engine(folder, EngineConfig(dtype="float32", page_size=16, max_cache_tokens=512, max_requests=3, max_batch_tokens=24, use_cuda_graphs=graphs))
    results = engine.generate(prompts, SamplingParams(max_tokens=20))
    for prompt, result in zip(prompts, results):
        assert result.generated_tokens == _plain_greedy(config, tensors, prompt, 20)
    again = engine.generate(prompts[:3], SamplingParams(max_tokens=20))       # pages come round again; shapes repeat, so graphs replay
    assert [r.generated_tokens for r in again] == [r.generated_tokens for r in results[:3]]
    if graphs:
        assert any(s.graph is not None for s in engine._sessions.values())
    engine.runner.cache.check()


@pytest.mark.gpu
def test_generation_in_bfloat16_and_the_command_line(folders, capsys):
    from tinyllama_inference_engine_b200 import generate
    from tinyllama_inference_engine_b200.cli import main

    rng = np.random.default_rng(2)
    prompts = [[int(t) for t in rng.integers(0, 53, size=n)] for n in (90, 12, 40)]
    first = generate(folders["plain_order"], prompts, max_tokens=24, dtype="bfloat16", page_size=16, max_cache_tokens=1024, max_requests=4, max_batch_tokens=64)
    second = generate(folders["plain_order"], prompts, max_tokens=24, dtype="bfloat16", page_size=16, max_cache_tokens=1024, max_requests=4, max_batch_tokens=64)
    assert first == second and all(len(tokens) == 24 for tokens in first)
    folder = folders["all"]
    config, tensors = load_plain(folder)
    prompt = [int(t) for t in np.random.default_rng(12).integers(0, config["vocab"], size=11)]
    text = ",".join(map(str, prompt))
    assert main(["generate", str(folder), text, "6", "--dtype", "float32", "--page-size", "16"]) == 0
    result = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert result["generated_tokens"] == _plain_greedy(config, tensors, prompt, 6) and result["prompt_tokens"] == 11
    assert main(["logits", str(folder), text, "--dtype", "float32"]) == 0
    logits = torch.tensor(json.loads(capsys.readouterr().out)["logits"])
    assert torch.allclose(logits, _logits(config, tensors, prompt)[-1], atol=3e-5 * float(logits.abs().max()))
