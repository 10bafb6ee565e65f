"""Typed configuration of Redasun, read from its own config.json keys.

``layers`` lists the layers one by one: ``{"type": "attention", "mixer": {heads, kv_heads, dim, vdim, scale, diff, rot: {base, dims}},
"mlp": null | {"kind": "dense", "ff": n} | {"kind": "moe", "expert": {ff}, "router": {experts, top, scale, groups: {count, keep}},
"shared": {ff} | null}}``.  Beside it: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` and optionally ``loop`` = {start, stop,
times} (layers start .. stop - 1 run ``times`` times in a row with the same weights).  Every size and constant is free; what the
design does not have is refused.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..config.model_config import as_float, as_int
from ..errors import ConfigError

MIXERS = ("attention",)
MLP_KINDS = ("dense", "moe")


def _mixer_sizes(index: int, mixer) -> dict:
    where = f"layers[{index}].mixer"
    if not isinstance(mixer, dict):
        raise ConfigError(f"{where} must be an object")
    heads = as_int(f"{where}.heads", mixer.get("heads"))
    kv_heads = as_int(f"{where}.kv_heads", mixer.get("kv_heads", heads))
    if heads % kv_heads != 0:
        raise ConfigError(f"{where}: heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
    dim = as_int(f"{where}.dim", mixer.get("dim"))
    vdim = as_int(f"{where}.vdim", mixer.get("vdim", dim))
    if dim > 256 or vdim > 256:
        raise ConfigError(f"{where}: dim ({dim}) and vdim ({vdim}) may be at most 256")
    diff = mixer.get("diff")
    if isinstance(diff, bool) or not isinstance(diff, (int, float)) or not 0.0 <= float(diff) < 1.0:
        raise ConfigError(f"{where}.diff must be a number in [0, 1), got {diff!r}")
    rot = mixer.get("rot")
    rot_sizes = {"base": 10000.0, "dims": 0}
    if rot is not None:
        if not isinstance(rot, dict):
            raise ConfigError(f"{where}.rot must be an object with base and dims, or null")
        dims = as_int(f"{where}.rot.dims", rot.get("dims", dim), minimum=0)
        if dims > dim or dims % 2:
            raise ConfigError(f"{where}: rot.dims ({dims}) must be even and at most dim ({dim})")
        rot_sizes = {"base": as_float(f"{where}.rot.base", rot.get("base")), "dims": dims}
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": as_float(f"{where}.scale", mixer.get("scale", dim ** -0.5)),
            "diff": float(diff), "rot": rot_sizes}


def _mlp_sizes(index: int, mlp):
    where = f"layers[{index}].mlp"
    if mlp is None:
        return None
    if not isinstance(mlp, dict) or mlp.get("kind", "dense") not in MLP_KINDS:
        raise ConfigError(f"{where} must be null or a feed-forward of kind {MLP_KINDS}, got {mlp!r}")
    if mlp.get("kind", "dense") == "dense":
        return {"kind": "dense", "ff": as_int(f"{where}.ff", mlp.get("ff"))}
    expert, router = mlp.get("expert"), mlp.get("router")
    if not isinstance(expert, dict) or not isinstance(router, dict):
        raise ConfigError(f"{where}: a mixture of experts has the objects expert and router")
    experts = as_int(f"{where}.router.experts", router.get("experts"))
    top = as_int(f"{where}.router.top", router.get("top"))
    groups = router.get("groups")
    if groups is None:
        groups = {"count": 1, "keep": 1}
    elif not isinstance(groups, dict):
        raise ConfigError(f"{where}.router.groups must be an object with count and keep, or absent")
    count = as_int(f"{where}.router.groups.count", groups.get("count", 1))
    keep = as_int(f"{where}.router.groups.keep", groups.get("keep", count))
    if experts % count or keep > count or top > keep * (experts // count):
        raise ConfigError(f"{where}.router: {experts} experts in {count} groups of which {keep} are kept cannot give {top} per token")
    shared = mlp.get("shared")
    if shared is not None:
        if not isinstance(shared, dict):
            raise ConfigError(f"{where}.shared must be an object with ff, or null")
        shared = {"ff": as_int(f"{where}.shared.ff", shared.get("ff"))}
    return {"kind": "moe", "expert": {"ff": as_int(f"{where}.expert.ff", expert.get("ff"))},
            "router": {"experts": experts, "top": top, "scale": as_float(f"{where}.router.scale", router.get("scale", 1.0)), "groups": {"count": count, "keep": keep}},
            "shared": shared}


@dataclass(frozen=True)
class RedasunConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: tuple                # one dictionary per layer: {"type", "mixer", "mlp"}, checked
    loop: dict | None = None     # {"start", "stop", "times"}
    architecture: str = "Redasun"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, data: dict) -> "RedasunConfig":
        if not isinstance(data, dict):
            raise ConfigError("config.json must hold a JSON object")
        missing = [key for key in ("vocab", "width", "norm", "layers") if key not in data]
        if missing:
            raise ConfigError("config.json lacks required keys: " + ", ".join(missing))
        if not isinstance(data["norm"], dict) or "eps" not in data["norm"]:
            raise ConfigError("config.json: norm must be an object with eps")
        if not isinstance(data["layers"], list) or not data["layers"]:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        layers = []
        for index, layer in enumerate(data["layers"]):
            if not isinstance(layer, dict):
                raise ConfigError(f"layers[{index}] must be an object")
            kind = layer.get("type")
            if kind not in MIXERS:
                raise ConfigError(f"layers[{index}].type must be one of {MIXERS}, got {kind!r}")
            layers.append({"type": kind, "mixer": _mixer_sizes(index, layer.get("mixer")), "mlp": _mlp_sizes(index, layer.get("mlp"))})
        loop = data.get("loop")
        if loop is not None:
            if not isinstance(loop, dict):
                raise ConfigError("config.json: loop must be an object or absent")
            loop = {"start": as_int("loop.start", loop.get("start"), minimum=0), "stop": as_int("loop.stop", loop.get("stop")), "times": as_int("loop.times", loop.get("times"))}
            if not loop["start"] < loop["stop"] <= len(layers):
                raise ConfigError(f"loop: start ({loop['start']}) < stop ({loop['stop']}) <= layers ({len(layers)}) does not hold")
        embedding = data.get("embedding") or {}
        return cls(vocab=as_int("vocab", data["vocab"]), width=as_int("width", data["width"]), norm_eps=as_float("norm.eps", data["norm"]["eps"]),
                   embedding_scale=as_float("embedding.scale", embedding.get("scale", 1.0)), layers=tuple(layers), loop=loop,
                   architecture=str(data.get("architecture", "Redasun")))

    def to_dict(self) -> dict:
        data = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "embedding": {"scale": self.embedding_scale}, "layers": [dict(layer) for layer in self.layers]}
        if self.loop is not None:
            data["loop"] = dict(self.loop)
        return data
