"""Typed configuration of Kilurax, read from its own config.json keys.

``layers`` lists the layers one by one: ``{"type": "parallel" | "hgrn2" | "delta", "mixer": {...sizes...}, "mlp": null | {"kind": "moe",
"expert": {ff}, "router": {experts, top}, "shared": {ff} | null}}``.  Beside it: ``vocab``, ``width``, ``norm`` = {eps, groups},
``residual_mult``, ``embedding`` = {scale, bigram: {buckets, mul_prev, mul_cur}}, ``canon`` = {taps}.  Every size and constant is free;
what the design does not have is refused.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..config.model_config import as_float, as_int
from ..errors import ConfigError

MIXERS = ("parallel", "hgrn2", "delta")


def _any_float(name: str, value) -> float:
    """A finite number of either sign (a scale of a branch may be negative or zero)."""
    if isinstance(value, bool) or not isinstance(value, (int, float)) or value != value or value in (float("inf"), float("-inf")):
        raise ConfigError(f"{name} must be a finite number, got {value!r}")
    return float(value)


def _object(where: str, value) -> dict:
    if not isinstance(value, dict):
        raise ConfigError(f"{where} must be an object")
    return value


def _heads(where: str, mixer: dict) -> tuple[int, int]:
    heads = as_int(f"{where}.heads", mixer.get("heads"))
    kv_heads = as_int(f"{where}.kv_heads", mixer.get("kv_heads", heads))
    if heads % kv_heads != 0:
        raise ConfigError(f"{where}: heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
    return heads, kv_heads


def _attention_sizes(where: str, mixer) -> dict:
    mixer = _object(where, mixer)
    heads, kv_heads = _heads(where, mixer)
    dim = as_int(f"{where}.dim", mixer.get("dim"))
    rot = mixer.get("rot")
    if rot is None:
        rot = {"base": 10000.0, "dims": 0}
    else:
        rot = _object(f"{where}.rot", rot)
        rot = {"base": as_float(f"{where}.rot.base", rot.get("base")), "dims": as_int(f"{where}.rot.dims", rot.get("dims", dim), minimum=0)}
    if rot["dims"] > dim or rot["dims"] % 2:
        raise ConfigError(f"{where}: rot.dims ({rot['dims']}) must be even and at most dim ({dim})")
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": as_int(f"{where}.vdim", mixer.get("vdim", dim)),
            "scale": as_float(f"{where}.scale", mixer.get("scale", dim ** -0.5)), "rot": rot}


def _ssd_sizes(where: str, mixer) -> dict:
    mixer = _object(where, mixer)
    heads = as_int(f"{where}.heads", mixer.get("heads"))
    groups = as_int(f"{where}.groups", mixer.get("groups", 1))
    vdim = as_int(f"{where}.vdim", mixer.get("vdim"))
    norm_groups = as_int(f"{where}.norm_groups", mixer.get("norm_groups", 1))
    if heads % groups or (heads * vdim) % norm_groups:
        raise ConfigError(f"{where}: heads ({heads}) must be a multiple of groups ({groups}), heads * vdim one of norm_groups ({norm_groups})")
    return {"heads": heads, "groups": groups, "vdim": vdim, "state": as_int(f"{where}.state", mixer.get("state")), "conv": as_int(f"{where}.conv", mixer.get("conv")),
            "norm_groups": norm_groups}


def _mixer_sizes(index: int, kind: str, mixer) -> dict:
    where = f"layers[{index}].mixer"
    mixer = _object(where, mixer)
    if kind == "parallel":
        return {"left": _attention_sizes(f"{where}.left", mixer.get("left")), "right": _ssd_sizes(f"{where}.right", mixer.get("right")),
                "left_scale": _any_float(f"{where}.left_scale", mixer.get("left_scale", 1.0)), "right_scale": _any_float(f"{where}.right_scale", mixer.get("right_scale", 1.0))}
    dim = as_int(f"{where}.dim", mixer.get("dim"))
    vdim = as_int(f"{where}.vdim", mixer.get("vdim", dim))
    if kind == "hgrn2":
        return {"heads": as_int(f"{where}.heads", mixer.get("heads")), "dim": dim, "vdim": vdim}
    heads, kv_heads = _heads(where, mixer)
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": as_int(f"{where}.conv", mixer.get("conv"))}


def _mlp_sizes(index: int, mlp):
    if mlp is None:
        return None
    where = f"layers[{index}].mlp"
    mlp = _object(where, mlp)
    if mlp.get("kind", "moe") != "moe":
        raise ConfigError(f"{where}.kind must be 'moe', got {mlp.get('kind')!r}")
    router, expert = _object(f"{where}.router", mlp.get("router")), _object(f"{where}.expert", mlp.get("expert"))
    experts, top = as_int(f"{where}.router.experts", router.get("experts")), as_int(f"{where}.router.top", router.get("top"))
    if top > experts:
        raise ConfigError(f"{where}.router: {top} of {experts} experts cannot be chosen")
    shared = mlp.get("shared")
    if shared is not None:
        shared = {"ff": as_int(f"{where}.shared.ff", _object(f"{where}.shared", shared).get("ff"))}
    return {"kind": "moe", "expert": {"ff": as_int(f"{where}.expert.ff", expert.get("ff"))}, "router": {"experts": experts, "top": top}, "shared": shared}


@dataclass(frozen=True)
class KiluraxConfig:
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    residual_mult: float
    embedding_scale: float
    layers: tuple                 # one dictionary per layer: {"type", "mixer", "mlp"}, checked
    bigram: dict | None = None    # {"buckets", "mul_prev", "mul_cur"}
    canon_taps: int = 0           # 0: no convolution in front of the sublayers
    architecture: str = "Kilurax"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, data: dict) -> "KiluraxConfig":
        if not isinstance(data, dict):
            raise ConfigError("config.json must hold a JSON object")
        missing = [key for key in ("vocab", "width", "norm", "layers") if key not in data]
        if missing:
            raise ConfigError("config.json lacks required keys: " + ", ".join(missing))
        if not isinstance(data["norm"], dict) or "eps" not in data["norm"]:
            raise ConfigError("config.json: norm must be an object with eps")
        if not isinstance(data["layers"], list) or not data["layers"]:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        width = as_int("width", data["width"])
        groups = as_int("norm.groups", data["norm"].get("groups", 1))
        if width % groups:
            raise ConfigError(f"width ({width}) must be a multiple of norm.groups ({groups})")
        layers = []
        for index, layer in enumerate(data["layers"]):
            layer = _object(f"layers[{index}]", layer)
            kind = layer.get("type")
            if kind not in MIXERS:
                raise ConfigError(f"layers[{index}].type must be one of {MIXERS}, got {kind!r}")
            layers.append({"type": kind, "mixer": _mixer_sizes(index, kind, layer.get("mixer")), "mlp": _mlp_sizes(index, layer.get("mlp"))})
        embedding = data.get("embedding") or {}
        bigram = _object("embedding", embedding).get("bigram")
        if bigram is not None:
            bigram = _object("embedding.bigram", bigram)
            bigram = {"buckets": as_int("embedding.bigram.buckets", bigram.get("buckets")), "mul_prev": as_int("embedding.bigram.mul_prev", bigram.get("mul_prev"), minimum=0),
                      "mul_cur": as_int("embedding.bigram.mul_cur", bigram.get("mul_cur"), minimum=0)}
        canon = data.get("canon")
        taps = 0 if canon is None else as_int("canon.taps", _object("canon", canon).get("taps"))
        return cls(vocab=as_int("vocab", data["vocab"]), width=width, norm_eps=as_float("norm.eps", data["norm"]["eps"]), norm_groups=groups,
                   residual_mult=_any_float("residual_mult", data.get("residual_mult", 1.0)), embedding_scale=_any_float("embedding.scale", embedding.get("scale", 1.0)),
                   layers=tuple(layers), bigram=bigram, canon_taps=taps, architecture=str(data.get("architecture", "Kilurax")))

    def to_dict(self) -> dict:
        data = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
                "residual_mult": self.residual_mult, "embedding": {"scale": self.embedding_scale}, "layers": [dict(layer) for layer in self.layers]}
        if self.bigram is not None:
            data["embedding"]["bigram"] = dict(self.bigram)
        if self.canon_taps:
            data["canon"] = {"taps": self.canon_taps}
        return data
