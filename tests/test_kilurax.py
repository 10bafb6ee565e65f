"""Kilurax through the framework against the plain implementation (plain_kilurax.py): configuration and names, cache groups, each
mechanism alone (the plain functions' own properties, the kernels by themselves, models of one kind of layer), and the engine's step
function under every way of cutting the work.  The ``gpu`` tests run the kernels; the others need no device."""
from __future__ import annotations

import json
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_kilurax
import trace_tools
from tinyllama_inference_engine_b200 import EngineConfig
from tinyllama_inference_engine_b200.cache import CacheManager
from tinyllama_inference_engine_b200.config import architecture_for, load_model_config
from tinyllama_inference_engine_b200.engine.batch import StepEntry
from tinyllama_inference_engine_b200.engine.runner import ModelRunner
from tinyllama_inference_engine_b200.errors import ConfigError
from tinyllama_inference_engine_b200.models import cache_needs, expected_tensors
from tinyllama_inference_engine_b200.models.kilurax_config import KiluraxConfig
from tinyllama_inference_engine_b200.weights import SafetensorsFile, write_random_model, write_safetensors


def _moe(experts, top, ff, shared=None):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}, "shared": None if shared is None else {"ff": shared}}


def _left(heads, kv, dim, vdim, rot, base=10000.0, scale=None):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else 1.5 * dim ** -0.5, "rot": {"base": base, "dims": rot}}


def _right(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def _parallel(left, right, mlp, scales=(0.8, 1.3)):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": scales[0], "right_scale": scales[1]}, "mlp": mlp}


def _hgrn2(heads, dim, vdim, mlp):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}, "mlp": mlp}


def _delta(heads, kv, dim, vdim, conv, mlp):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


def _config(width, vocab, layers, groups=2, taps=3, mult=0.7, eps=1e-5, embed_scale=4.0, bigram=(211, 31, 5)):
    data = {"architecture": "Kilurax", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups}, "residual_mult": mult,
            "embedding": {"scale": embed_scale}, "layers": layers}
    if bigram:
        data["embedding"]["bigram"] = dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))
    if taps:
        data["canon"] = {"taps": taps}
    return data


# Sizes that agree nowhere: grouped and ungrouped heads, key and value widths equal and not, rotations of the whole head, of a part and of
# nothing, state-space layers with shared and separate groups, norms over one group and several, experts one per token, several and all,
# with and without a shared expert, layers without a feed-forward, every kind of layer first and last.
CONFIGS = {
    "all": (_config(64, 97, [_parallel(_left(4, 2, 16, 32, 8), _right(4, 16, 16, 2, 3, 2), _moe(6, 2, 24, shared=40)), _hgrn2(2, 16, 32, None),
                             _delta(4, 2, 16, 16, 3, _moe(4, 1, 16)), _parallel(_left(2, 2, 32, 16, 32, base=500.0), _right(2, 32, 8, 1, 4, 1), _moe(5, 3, 8, shared=8), scales=(1.2, 0.5)),
                             _hgrn2(4, 8, 8, _moe(3, 3, 16, shared=24))], groups=4, taps=4), 3),
    "recurrent_first": (_config(48, 61, [_delta(2, 2, 24, 8, 2, _moe(4, 2, 32, shared=16)), _hgrn2(3, 16, 16, _moe(2, 1, 8)), _parallel(_left(6, 2, 8, 16, 0), _right(3, 16, 24, 3, 2, 3), None)],
                                groups=3, taps=2, mult=1.5, eps=1e-6, embed_scale=9.0, bigram=(53, 3, 11)), 5),
    # what another model may make 1 or leave out: one norm group, a convolution of one tap, no second table, all scales 1, every expert chosen
    "ones": (_config(40, 53, [_hgrn2(1, 40, 40, _moe(3, 3, 24)), _parallel(_left(5, 5, 8, 8, 2, base=50.0, scale=1.0), _right(1, 40, 16, 1, 1, 1), _moe(2, 1, 16, shared=8), scales=(1.0, 1.0)),
                              _delta(1, 1, 8, 40, 1, None)], groups=1, taps=1, mult=1.0, embed_scale=1.0, bigram=None), 9),
    # nothing a multiple of 8: the width, the vocabulary, the feed-forwards, the heads' widths, the states
    "odd": (_config(44, 37, [_parallel(_left(3, 1, 12, 10, 6), _right(2, 22, 12, 2, 5, 2), _moe(6, 2, 10, shared=6)), _delta(3, 1, 10, 6, 4, _moe(5, 2, 50)), _hgrn2(2, 10, 22, None)],
                    groups=2, taps=5, bigram=(17, 1000003, 7)), 8),
}
LENGTHS = {"all": [1, 9, 70, 150, 33, 64, 17], "recurrent_first": [3, 40, 100, 64, 7], "ones": [2, 130, 65, 16], "odd": [70, 3, 33, 18]}
TOLERANCE = {"float32": 3e-5, "bfloat16": 2.5e-2}     # 32-bit: of a row's largest difference; bfloat16: of its root mean square over the vocabulary
RMS = {"float32": False, "bfloat16": True}
SHARP = {"float32": 1.0, "bfloat16": 3.0}             # models whose weights were changed so that far tokens decide: see the tests that use it
# bfloat16 rounds what the routers read, and of some hundred tokens a few then choose another expert than the plain implementation does; such
# a row (and, through the recurrent states, rows behind it) differs by many times the rounding.  32-bit rows are all held to their bound;
# in bfloat16 a share of the rows may lie beyond it while the median row lies within a third of it (trace_tools.run_and_compare).
LOOSE_ROWS = {"float32": 0.0, "bfloat16": 0.25}


def load_plain(folder, dtype=torch.float64):
    config = json.loads((folder / "config.json").read_text())
    file = SafetensorsFile(folder / "model.safetensors")
    tensors = {name: file.tensor(name).clone().to(dtype) for name in file.names()}
    file.close()
    return config, tensors


def _logits(config, tensors, tokens):
    return plain_kilurax.forward(tokens, tensors, config)[0].float()


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("kilurax")
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
    assert architecture.name == "Kilurax" and isinstance(config, KiluraxConfig)
    assert KiluraxConfig.from_dict(config.to_dict()) == config
    assert config.layers[1]["mlp"] is None and config.canon_taps == 4 and config.norm_groups == 4 and config.bigram == {"buckets": 211, "mul_prev": 31, "mul_cur": 5}
    spec = architecture.build_spec(config)
    names = {t.name: tuple(t.shape) for t in expected_tensors(spec)}
    assert names["embed"] == (97, 64) and names["bigram"] == (212, 64) and names["embed.norm"] == (64,) and names["final.norm"] == (64,) and names["head"] == (97, 64)
    assert names["l0.mix.left.q"] == (64, 64) and names["l0.mix.left.k"] == (32, 64) and names["l0.mix.left.v"] == (64, 64) and names["l0.mix.left.o"] == (64, 128)
    assert names["l0.mix.left.q.b"] == (64,) and names["l0.mix.left.o.b"] == (64,)
    assert names["l0.mix.right.in"] == (64 + 64 + 32 + 32 + 4, 64) and names["l0.mix.right.conv"] == (128, 3) and names["l0.mix.right.conv.b"] == (128,)
    assert names["l0.mix.right.D"] == (4,) and names["l0.mix.right.norm"] == (64,) and names["l0.mix.right.o"] == (64, 64)
    assert names["l0.canon1"] == (64, 4) and names["l0.canon2"] == (64, 4) and names["l0.norm1b"] == (64,) and names["l0.norm2b"] == (64,)
    assert names["l1.mix.q"] == (32, 64) and names["l1.mix.f.b"] == (32,) and names["l1.mix.lower"] == (32,) and names["l1.mix.v"] == (64, 64) and names["l1.mix.norm"] == (32,)
    assert "l1.norm2" not in names and "l1.canon2" not in names and "l1.mlp.router" not in names
    assert names["l2.mix.q.conv"] == (32, 3) and names["l2.mix.v.conv"] == (64, 3) and names["l2.mix.b"] == (4, 64) and names["l2.mix.a"] == (4, 64) and names["l2.mix.dt_bias"] == (4,)
    assert names["l2.mix.g"] == (64, 64) and names["l2.mlp.e3.down"] == (64, 16) and names["l2.mlp.router"] == (4, 64) and "l2.mlp.shared.gate" not in names
    assert names["l3.mlp.shared.up"] == (8, 64) and "l0.mlp.correction" not in names
    ones = architecture.build_spec(KiluraxConfig.from_dict(CONFIGS["ones"][0]))
    assert not any(t.name == "bigram" or "canon" in t.name and t.shape[1] != 1 for t in expected_tensors(ones))


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="lstm"), "type"),
    (lambda c: c["layers"][0].update(mlp={"kind": "dense", "ff": 8}), "kind"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(groups=3), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "experts"),
    (lambda c: c["norm"].update(groups=5), "norm.groups"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_configuration_refuses_what_the_design_lacks(change, message):
    data = json.loads(json.dumps(CONFIGS["all"][0]))
    change(data)
    with pytest.raises(ConfigError, match=message):
        KiluraxConfig.from_dict(data)


def test_cache_groups_hold_pages_and_state_of_one_layer():
    """A layer with attention beside a state-space layer is in a page group and in a state group; the embedding keeps one word per request;
    the convolutions' inputs lie behind the mixer's own state."""
    from tinyllama_inference_engine_b200 import ops

    architecture = architecture_for(CONFIGS["all"][0])
    needs = cache_needs(architecture.build_spec(architecture.config_class.from_dict(CONFIGS["all"][0])))
    assert needs[-1].kind == "state" and needs[-1].state_shape == (1,)
    assert needs[0].kind == "pages" and needs[0].page_planes() == ((2, 16), (2, 32))
    ssd = ops.delta_state_words(4, 16, 16, 64 + 2 * 2 * 16, 3)[0]
    assert needs[0].state_shape == (ssd + 2 * 3 * 64,)                       # the mixer's matrices and inputs, then both convolutions' three inputs of 64
    assert needs[1].kind == "state" and needs[1].state_shape == (ops.delta_state_words(2, 16, 32, 0, 1)[0] + 3 * 64,)   # no feed-forward: one convolution
    manager = CacheManager(needs, page_size=16, num_pages=40, max_requests=2, max_positions=4096, device="cpu")
    assert sorted((g.need.page_planes(), g.streams) for g in manager.page_groups) == [(((2, 16), (2, 32)), [0]), (((2, 32), (2, 16)), [3])]
    assert sorted(s for g in manager.state_groups for s in g.streams) == [-1, 0, 1, 2, 3, 4]      # layers whose states are of one size share a group
    record = manager.admit("a")
    manager.reserve("a", 20)
    caches = manager.layer_caches([torch.tensor(manager.block_table_rows(g, ["a"]), dtype=torch.int32) for g in manager.page_groups])
    assert caches[0].state.shape == (2, needs[0].state_shape[0]) and caches[0].block_table.shape[0] == 1 and len(caches[0].plane_pages) == 2
    assert caches[1].block_table is None and caches[-1].state.shape == (2, 1) and record.slot in (0, 1)


# --- the plain implementation's own mechanisms --------------------------------------------------------------------------------------
def test_plain_norm_convolution_and_embedding():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(5, 12, generator=g, dtype=torch.float64)
    w = torch.randn(12, generator=g, dtype=torch.float64)
    one = plain_kilurax.grouped_rms_norm(x, w, 1, 1e-6)
    assert torch.allclose(one, x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-6) * w)
    three = plain_kilurax.grouped_rms_norm(x, w, 3, 1e-6)
    assert torch.allclose(three[:, 4:8], plain_kilurax.grouped_rms_norm(x[:, 4:8], w[4:8], 1, 1e-6)) and not torch.allclose(three, one)
    taps = torch.randn(12, 3, generator=g, dtype=torch.float64)
    y = plain_kilurax.causal_conv(x, taps)
    assert torch.allclose(y[0], taps[:, 2] * x[0]) and torch.allclose(y[1], taps[:, 2] * x[1] + taps[:, 1] * x[0])      # zeros before the start
    assert torch.allclose(y[4], taps[:, 2] * x[4] + taps[:, 1] * x[3] + taps[:, 0] * x[2])
    cfg = {"embedding": {"scale": 3.0, "bigram": {"buckets": 7, "mul_prev": 5, "mul_cur": 3}}, "norm": {"groups": 2, "eps": 1e-6}}
    P = {"embed": torch.randn(10, 12, generator=g, dtype=torch.float64), "bigram": torch.randn(8, 12, generator=g, dtype=torch.float64), "embed.norm": torch.ones(12, dtype=torch.float64)}
    rows = plain_kilurax.embed([4, 9, 9], P, cfg)
    assert torch.allclose(rows[0], plain_kilurax.grouped_rms_norm((P["embed"][4] * 3.0 + P["bigram"][7])[None], P["embed.norm"], 2, 1e-6)[0])    # the first token: the last row
    assert torch.allclose(rows[2], plain_kilurax.grouped_rms_norm((P["embed"][9] * 3.0 + P["bigram"][(9 * 5 + 9 * 3) % 7])[None], P["embed.norm"], 2, 1e-6)[0])
    assert not torch.allclose(rows[1], rows[2])     # the same token after another one


def test_plain_recurrences_and_experts():
    g = torch.Generator().manual_seed(2)
    h = torch.randn(7, 12, generator=g, dtype=torch.float64)
    m = {"heads": 2, "dim": 4, "vdim": 3}
    P = {"m.q": torch.randn(8, 12, generator=g, dtype=torch.float64), "m.f": torch.randn(8, 12, generator=g, dtype=torch.float64), "m.f.b": torch.zeros(8, dtype=torch.float64),
         "m.lower": torch.full((8,), 0.25, dtype=torch.float64), "m.v": torch.randn(6, 12, generator=g, dtype=torch.float64), "m.norm": torch.ones(3, dtype=torch.float64),
         "m.o": torch.eye(12, 6, dtype=torch.float64)}
    out = plain_kilurax.hgrn2(h, P, "m", m, 1e-6)
    # the first token: S = (1 - f) v^T, so o = ((1 - f) . q) v and every head's normalised output is +-v / rms(v)
    v0 = (h[0] @ P["m.v"].T).reshape(2, 3)
    assert torch.allclose(out[0, :6].reshape(2, 3).abs(), (v0 / torch.sqrt((v0 * v0).mean(-1, keepdim=True) + 1e-6)).abs(), atol=1e-4)
    # a lower bound of one forgets nothing and writes nothing: the output is that of an empty state
    P["m.lower"] = torch.ones(8, dtype=torch.float64)
    assert float(plain_kilurax.hgrn2(h, P, "m", m, 1e-6).abs().max()) == 0.0
    # experts: the score multiplies what the expert reads, which is not the same as multiplying what it returns
    E = {"f.router": torch.randn(3, 12, generator=g, dtype=torch.float64)}
    for e in ("e0", "e1", "e2", "shared"):
        E.update({f"f.{e}.gate": torch.randn(5, 12, generator=g, dtype=torch.float64), f"f.{e}.up": torch.randn(5, 12, generator=g, dtype=torch.float64),
                  f"f.{e}.down": torch.randn(12, 5, generator=g, dtype=torch.float64)})
    mlp = {"router": {"experts": 3, "top": 1}, "shared": {"ff": 5}}
    got = plain_kilurax.routed_experts(h[:1], E, "f", mlp)
    scores = torch.sigmoid(h[0] @ E["f.router"].T)
    best = int(scores.argmax())
    want = plain_kilurax.expert(scores[best] * h[:1], E, f"f.e{best}") + plain_kilurax.expert(h[:1], E, "f.shared")
    assert torch.allclose(got, want) and not torch.allclose(got, scores[best] * plain_kilurax.expert(h[:1], E, f"f.e{best}") + plain_kilurax.expert(h[:1], E, "f.shared"))
    x = torch.randn(5, 3, 8, generator=g, dtype=torch.float64)
    turned = plain_kilurax.rotate(x, 4, 100.0)
    assert torch.equal(turned[..., 4:], x[..., 4:]) and torch.equal(turned[0], x[0]) and torch.allclose((turned * turned).sum(-1), (x * x).sum(-1))
    assert torch.allclose(turned[2, 0, 0], x[2, 0, 0] * np.cos(2.0) - x[2, 0, 2] * np.sin(2.0))          # column 0 turns with column 2 = dims / 2


# --- kernels by themselves ------------------------------------------------------------------------------------------------------------
def _ctx(pieces, slots):
    """The context of a step that brings ``n`` rows from position ``a`` of a request for every (a, n) in ``pieces``."""
    lens = [n for _, n in pieces]
    starts = np.concatenate([[0], np.cumsum(lens)])
    to = lambda values: torch.tensor(np.asarray(values), dtype=torch.int32).cuda()  # noqa: E731
    return SimpleNamespace(num_seqs=len(pieces), num_tokens=int(starts[-1]), seq_starts=to(starts), state_slots=to(slots),
                           token_seq=to(np.repeat(np.arange(len(pieces)), lens)), positions=to(np.concatenate([np.arange(a, a + n) for a, n in pieces])),
                           max_q_len=max(lens), max_seq_len=max(a + n for a, n in pieces), token_ids=None)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,atol", [(torch.float32, 3e-6), (torch.bfloat16, 1.2e-2)])
@pytest.mark.parametrize("width,groups", [(44, 2), (256, 4), (96, 3), (120, 1), (1000, 5)])
def test_grouped_norm_kernel(dtype, atol, width, groups):
    from tinyllama_inference_engine_b200 import ops

    g = torch.Generator().manual_seed(width)
    stream = torch.randn(9, width, generator=g) * 3.0 + 1.0
    y = (torch.randn(9, width, generator=g) * 2.0 - 0.5).to(dtype)
    y[:, : width // groups] *= 30.0     # one part far larger than the others: statistics over the whole row would show
    post, following = 1 + 0.1 * torch.randn(width, generator=g), 1 + 0.1 * torch.randn(width, generator=g)
    want_stream = stream.double() + plain_kilurax.grouped_rms_norm(y.double(), post.double(), groups, 1e-5)
    want_out = plain_kilurax.grouped_rms_norm(want_stream, following.double(), groups, 1e-5)
    residual = stream.cuda()
    out = torch.zeros(9, width, dtype=dtype, device="cuda")
    ops.branch_norm(residual, y.cuda(), post.cuda(), following.cuda(), out, 1e-5, False, groups=groups)
    assert float((residual.cpu().double() - want_stream).abs().max()) <= 3e-6 * float(want_stream.abs().max())
    assert float((out.cpu().double() - want_out).abs().max()) <= atol * float(want_out.abs().max())
    rows = torch.tensor([7, 2, 2], dtype=torch.int32).cuda()
    some = torch.zeros(3, width, dtype=dtype, device="cuda")
    ops.branch_norm(residual, None, None, following.cuda(), some, 1e-5, False, rows, groups=groups)
    assert torch.equal(some.cpu(), out.cpu()[[7, 2, 2]])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("channels,taps", [(44, 3), (64, 5), (10, 2), (24, 1)])
def test_input_convolution_and_pair_embedding_keep_what_came_before(dtype, channels, taps):
    """Two requests in steps of unequal portions (down to one row, fewer than the taps) against the whole sequences; slots used in another order."""
    from tinyllama_inference_engine_b200 import ops

    g = torch.Generator().manual_seed(channels)
    whole = [torch.randn(n, channels, generator=g).to(dtype) for n in (23, 9)]
    weight = torch.randn(channels, taps, generator=g)
    want = [w.double() + plain_kilurax.causal_conv(w.double(), weight.double()) for w in whole]
    state = torch.full((3, 7 + (taps - 1) * channels), float("nan"), device="cuda")
    state[[2, 0]] = 0.0
    at, got = [0, 0], [[], []]
    for cut in ([(0, 5), (1, 1)], [(0, 1), (1, 2)], [(1, 6)], [(0, 2), (0, 0)], [(0, 15)]):
        pieces = [(r, n) for r, n in cut if n > 0]
        ctx = _ctx([(at[r], n) for r, n in pieces], [2 if r == 0 else 0 for r, _ in pieces])
        x = torch.cat([whole[r][at[r] : at[r] + n] for r, n in pieces]).cuda()
        out = torch.zeros_like(x)
        ops.conv_residual(x, weight.cuda(), state, 7, ctx, out)
        for (r, n), rows in zip(pieces, out.cpu().double().split([n for _, n in pieces])):
            got[r].append(rows)
            at[r] += n
    tolerance = 1e-5 if dtype == torch.float32 else 3e-2
    for r in range(2):
        assert float((torch.cat(got[r]) - want[r][: at[r]]).abs().max()) <= tolerance * float(want[r].abs().max())
    assert bool(torch.isnan(state[1]).all()) and bool(torch.isnan(state[:, :7][[0, 2]]).logical_not().all())
    # the embedding: token rows, pair rows by (token before, token), the first token's own row, the token before a step kept per request
    vocab, buckets = 19, 11
    table, pairs, weight = torch.randn(vocab, channels, generator=g).to(dtype), torch.randn(buckets + 1, channels, generator=g).to(dtype), 1 + 0.1 * torch.randn(channels, generator=g)
    cfg = {"embedding": {"scale": 2.5, "bigram": {"buckets": buckets, "mul_prev": 100003, "mul_cur": 7}}, "norm": {"groups": 2, "eps": 1e-5}}
    tokens = [[int(t) for t in torch.randint(0, vocab, (n,), generator=g)] for n in (12, 5)]
    P = {"embed": table.double(), "bigram": pairs.double(), "embed.norm": weight.double()}
    want = [plain_kilurax.embed(t, P, cfg) for t in tokens]
    word = torch.zeros(3, 4, device="cuda")
    at, got = [0, 0], [[], []]
    for cut in ([(0, 4), (1, 1)], [(1, 1)], [(0, 1), (1, 3)], [(0, 7)]):
        ctx = _ctx([(at[r], n) for r, n in cut], [1 if r == 0 else 2 for r, _ in cut])
        ctx.token_ids = torch.tensor([t for r, n in cut for t in tokens[r][at[r] : at[r] + n]], dtype=torch.int32).cuda()
        residual = torch.zeros(ctx.num_tokens, channels, device="cuda")
        ops.pair_embedding(table.cuda(), pairs.cuda(), ctx, word, 3, weight.cuda(), 1e-5, 2.5, residual, buckets, 100003, 7, 2)
        for (r, n), rows in zip(cut, residual.cpu().double().split([n for _, n in cut])):
            got[r].append(rows)
            at[r] += n
    for r in range(2):
        assert float((torch.cat(got[r]) - want[r]).abs().max()) <= 1e-5 * float(want[r].abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["parallel", "hgrn2", "delta"])
def test_models_of_one_kind_of_layer(tmp_path, kind, dtype):
    """Each mixer alone in a model of two layers, sizes unlike the other tests', whole and token by token."""
    layer = {"parallel": lambda mlp: _parallel(_left(2, 1, 24, 8, 12, base=77.0), _right(6, 8, 20, 3, 3, 2), mlp, scales=(-0.6, 1.1)),
             "hgrn2": lambda mlp: _hgrn2(3, 20, 12, mlp), "delta": lambda mlp: _delta(6, 3, 12, 20, 5, mlp)}[kind]
    config = _config(72, 45, [layer(None), layer(_moe(3, 2, 12, shared=20))], groups=3, taps=0 if kind == "hgrn2" else 2, mult=0.9)   # one of them without the convolutions
    folder = write_random_model(tmp_path / kind, config, seed=13)
    config, tensors = load_plain(folder)
    requests = trace_tools.make_requests(45, [50, 3, 21], seed=5)
    full = {rid: _logits(config, tensors, tokens) for rid, tokens in requests.items()}
    scale = max(float(v.abs().max()) for v in full.values())
    for steps in (trace_tools.whole(requests), trace_tools.tail_decode(requests, tail=20), trace_tools.portions(requests)):
        trace_tools.run_and_compare(_runner(folder, dtype), steps, full, atol=TOLERANCE[dtype] * scale, over_vocabulary=RMS[dtype], allowed_over=LOOSE_ROWS[dtype])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_widest_heads_and_longest_taps(tmp_path, dtype):
    """Key widths and states of 200 and 256 channels (the recurrence's widest form, whose staged rows need more shared memory than a kernel gets unasked),
    convolutions of seven taps, an attention head of 144."""
    config = _config(72, 45, [_hgrn2(1, 200, 24, None), _delta(2, 1, 256, 16, 7, _moe(3, 1, 12)), _parallel(_left(2, 1, 144, 8, 0), _right(2, 16, 200, 1, 7, 1), None)],
                     groups=2, taps=7)
    folder = write_random_model(tmp_path / "wide", config, seed=4)
    config, tensors = load_plain(folder)
    requests = trace_tools.make_requests(45, [40, 9], seed=6)
    full = {rid: _logits(config, tensors, tokens) for rid, tokens in requests.items()}
    scale = max(float(v.abs().max()) for v in full.values())
    for steps in (trace_tools.whole(requests), trace_tools.tail_decode(requests, tail=12), trace_tools.portions(requests)):
        trace_tools.run_and_compare(_runner(folder, dtype), steps, full, atol=TOLERANCE[dtype] * scale, over_vocabulary=RMS[dtype], allowed_over=LOOSE_ROWS[dtype])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,atol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("tokens,experts,top,width,ff,shared", [(5, 6, 2, 44, 10, True), (70, 8, 3, 64, 24, True), (300, 4, 1, 32, 16, False), (1, 3, 3, 24, 8, False),
                                                                (700, 6, 3, 136, 200, True)])
def test_experts_that_read_their_token_times_its_score(dtype, atol, tokens, experts, top, width, ff, shared):
    """Scores that are not normalised, and the score on the expert's input: the plain sum of expert(w x) + shared(x)."""
    from tinyllama_inference_engine_b200 import ops

    g = torch.Generator().manual_seed(tokens + experts)
    x = torch.randn(tokens, width, generator=g).to(dtype)
    router = torch.randn(experts, width, generator=g) * 2.0 * width ** -0.5
    gate_up = (torch.randn(experts, 2 * ff, width, generator=g) * width ** -0.5).to(dtype)
    down = (torch.randn(experts, width, ff, generator=g) * ff ** -0.5).to(dtype)
    ids = torch.zeros(tokens, top, dtype=torch.int32, device="cuda")
    weights = torch.zeros(tokens, top, device="cuda")
    ops.moe_route(x.cuda(), router.cuda(), None, ids, weights, 1, 1, 1.0, normalize=False)
    scores = torch.sigmoid(x.double() @ router.double().T)
    order = torch.argsort(-scores, dim=1, stable=True)[:, :top]
    close = (scores.gather(1, order)[:, -1] - scores.gather(1, torch.argsort(-scores, dim=1, stable=True)[:, top : top + 1]).squeeze(1)).abs() < 1e-5 if top < experts else torch.zeros(tokens, dtype=torch.bool)
    rows = (~close).nonzero().squeeze(1)
    assert len(rows) >= tokens - 2 and torch.equal(ids.cpu()[rows].long(), order[rows])
    assert torch.allclose(weights.cpu()[rows].double(), scores.gather(1, order)[rows], atol=1e-5)      # the scores themselves: they need not sum to one
    branch = torch.randn(tokens, width, generator=g).to(dtype) if shared else None
    want = torch.zeros(tokens, width, dtype=torch.float64) if branch is None else branch.double().clone()
    for t in range(tokens):
        for k in range(top):
            e, w = int(ids[t, k]), float(weights[t, k])
            z = gate_up[e].double() @ (w * x[t].double())
            want[t] += down[e].double() @ (z[:ff] * torch.sigmoid(z[:ff]) * z[ff:])
    got = torch.zeros(tokens, width, dtype=dtype, device="cuda")
    ops.moe_experts(x.cuda(), gate_up.cuda(), down.cuda(), ids, weights, None if branch is None else branch.cuda(), got, "silu", weight_input=True)
    assert float((got.cpu().double() - want).abs().max()) <= atol * max(1.0, float(want.abs().max()))


# --- the engine on the GPU under every way of cutting the work ---------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", list(CONFIGS))
def test_engine_matches_plain_under_every_schedule(cases, key, dtype):
    """Whole prompts, a tail decoded token by token, portions down to two tokens, and four live requests mixed in a pool that makes
    pages and state slots come round again (freed pages are poisoned with NaN)."""
    folder, requests, full, scale = cases[key]
    for name, (steps, pool) in _schedules(requests).items():
        runner = _runner(folder, dtype, max_tokens=pool)
        trace_tools.run_and_compare(runner, steps, full, atol=TOLERANCE[dtype] * scale, over_vocabulary=RMS[dtype], allowed_over=LOOSE_ROWS[dtype])
        runner.cache.check()
        assert not runner.cache.records, name
        if name == "mixed":
            assert all(g.pool.reuses > 0 for g in runner.cache.page_groups)


@pytest.mark.gpu
def test_layer_outputs_match_the_plain_trace(cases):
    folder, requests, full, scale = cases["all"]
    config, tensors = load_plain(folder)
    tokens = requests["r4"]
    want = plain_kilurax.forward(tokens, tensors, config)[1]
    trace = {}
    _runner(folder, "float32").step([StepEntry("a", tokens, [0])], trace=trace)
    assert len(trace) == len(want) == 5
    for index, layer in enumerate(want):
        assert float((trace[f"layer{index}.output"].cpu().double() - layer).abs().max()) <= 3e-5 * float(layer.abs().max()), index


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
def test_far_keys_long_memories_and_first_tokens_decide(folders, dtype):
    """A large score scale lets single keys win a row, hundreds of tokens back and across page borders; decays close to one and lower bounds
    close to one make the recurrent states remember as far; a heavy second table makes the token before count.  A lost key, a lost or
    stale state, a rotation by the wrong position or a wrong token before then moves the logits far beyond the tolerance, in portions,
    in decoded tokens and in mixed batches."""
    def edit(tensors):
        for name in tensors:
            if name.endswith(".A_log"):
                tensors[name] = torch.full_like(tensors[name], -7.0)
            if name.endswith(".lower"):
                tensors[name] = torch.full_like(tensors[name], 0.992)
            if name == "bigram":
                tensors[name] = tensors[name] * 3.0

    def sharper(config):
        for layer in config["layers"]:
            if layer["type"] == "parallel":
                layer["mixer"]["left"]["scale"] = 2.0

    folder = _sharpened(folders["all"], "sharp", edit, sharper)
    config, tensors = load_plain(folder)
    requests = trace_tools.make_requests(config["vocab"], [400, 70, 33], seed=17)
    full = {rid: _logits(config, tensors, tokens) for rid, tokens in requests.items()}
    scale = max(float(v.abs().max()) for v in full.values())
    early = [(t + 1) % config["vocab"] if 10 <= i < 60 else t for i, t in enumerate(requests["r0"])]       # 340 tokens and more back
    assert float((_logits(config, tensors, early)[-1] - full["r0"][-1]).abs().max()) > 50 * TOLERANCE["float32"] * scale
    first = [(requests["r0"][0] + 1) % config["vocab"]] + requests["r0"][1:]
    assert float((_logits(config, tensors, first)[100:] - full["r0"][100:]).abs().max()) > 50 * TOLERANCE["float32"] * scale      # the first token shows hundreds of tokens on
    # states that forget nothing also keep every token's rounding: bfloat16 gets a wider bound here, 32-bit the usual one
    for steps in (trace_tools.tail_decode(requests, tail=40), trace_tools.portions(requests), trace_tools.mixed(requests, seed=4, max_portion=90)[0]):
        trace_tools.run_and_compare(_runner(folder, dtype, max_tokens=2048), steps, full, atol=SHARP[dtype] * TOLERANCE[dtype] * scale, over_vocabulary=RMS[dtype], allowed_over=LOOSE_ROWS[dtype])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_only_the_state_space_layer_or_only_the_attention_remembers(folders, dtype):
    """With one side of the parallel mixer weighed out the other side alone carries what lies far back: its cache or its state must be right by itself."""
    for side in ("left_scale", "right_scale"):
        def one_side(config, side=side):
            for layer in config["layers"]:
                if layer["type"] == "parallel":
                    layer["mixer"][side] = 1e-3
                    layer["mixer"]["left"]["scale"] = 1.5

        def edit(tensors):
            for name in tensors:
                if name.endswith("right.A_log"):
                    tensors[name] = torch.full_like(tensors[name], -6.0)

        folder = _sharpened(folders["recurrent_first"], side, edit, one_side)
        config, tensors = load_plain(folder)
        requests = trace_tools.make_requests(config["vocab"], [200, 45], seed=3)
        full = {rid: _logits(config, tensors, tokens) for rid, tokens in requests.items()}
        scale = max(float(v.abs().max()) for v in full.values())
        for steps in (trace_tools.tail_decode(requests, tail=40), trace_tools.portions(requests)):
            trace_tools.run_and_compare(_runner(folder, dtype, max_tokens=2048), steps, full, atol=SHARP[dtype] * TOLERANCE[dtype] * scale, over_vocabulary=RMS[dtype], allowed_over=LOOSE_ROWS[dtype])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_other_page_sizes(cases, dtype):
    """150 tokens decoded one by one behind a prompt, with pages of 64 and of 32 tokens."""
    folder, requests, full, scale = cases["recurrent_first"]
    some = {rid: requests[rid] for rid in ("r2", "r3")}
    more = dict(some, long=trace_tools.make_requests(61, [260], seed=5)["r0"])
    config, tensors = load_plain(folder)
    full = dict(full, long=_logits(config, tensors, more["long"]))
    for page_size in (64, 32):
        trace_tools.run_and_compare(_runner(folder, dtype, max_tokens=2048, page_size=page_size), trace_tools.tail_decode(more, tail=150), full,
                                    atol=TOLERANCE[dtype] * scale, over_vocabulary=RMS[dtype], allowed_over=LOOSE_ROWS[dtype])


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
    graphs or not; the token before a decoded one is the one the device chose).  32-bit, so that the plain choice is the engine's."""
    from tinyllama_inference_engine_b200 import Engine, SamplingParams

    folder = folders["all"]
    config, tensors = load_plain(folder)
    rng = np.random.default_rng(31)
    prompts = [[int(t) for t in rng.integers(0, config["vocab"], size=n)] for n in (50, 3, 21, 34, 8)]
    engine = Engine(folder, EngineConfig(dtype="float32", page_size=16, max_cache_tokens=512, max_requests=3, max_batch_tokens=24, use_cuda_graphs=graphs))
    results = engine.generate(prompts, SamplingParams(max_tokens=20))
    for prompt, result in zip(prompts, results):
        assert result.generated_tokens == _plain_greedy(config, tensors, prompt, 20)
    again = engine.generate(prompts[:3], SamplingParams(max_tokens=20))       # pages and slots come round again; shapes repeat, so graphs replay
    assert [r.generated_tokens for r in again] == [r.generated_tokens for r in results[:3]]
    if graphs:
        assert any(s.graph is not None for s in engine._sessions.values())
    engine.runner.cache.check()


@pytest.mark.gpu
def test_generation_in_bfloat16_and_the_command_line(folders, capsys):
    from tinyllama_inference_engine_b200 import generate
    from tinyllama_inference_engine_b200.cli import main

    rng = np.random.default_rng(2)
    prompts = [[int(t) for t in rng.integers(0, 61, size=n)] for n in (90, 12, 40)]
    first = generate(folders["recurrent_first"], prompts, max_tokens=24, dtype="bfloat16", page_size=16, max_cache_tokens=1024, max_requests=4, max_batch_tokens=64)
    second = generate(folders["recurrent_first"], prompts, max_tokens=24, dtype="bfloat16", page_size=16, max_cache_tokens=1024, max_requests=4, max_batch_tokens=64)
    assert first == second and all(len(tokens) == 24 for tokens in first)
    folder = folders["odd"]
    config, tensors = load_plain(folder)
    prompt = [int(t) for t in np.random.default_rng(12).integers(0, config["vocab"], size=11)]
    text = ",".join(map(str, prompt))
    assert main(["generate", str(folder), text, "6", "--dtype", "float32", "--page-size", "16"]) == 0
    result = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert result["generated_tokens"] == _plain_greedy(config, tensors, prompt, 6) and result["prompt_tokens"] == 11
    assert main(["logits", str(folder), text, "--dtype", "float32"]) == 0
    logits = torch.tensor(json.loads(capsys.readouterr().out)["logits"])
    assert torch.allclose(logits, _logits(config, tensors, prompt)[-1], atol=3e-5 * float(logits.abs().max()))
