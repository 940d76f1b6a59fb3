"""Typed configuration of the Naditar design, read from its own config.json keys.

config.json names every size and every constant that differs between models of the design:
  architecture        "Naditar"
  vocab, width        vocabulary and width of the residual stream
  norm.eps            the one epsilon of all root-mean-square norms
  layers[i]           type ("lightning" | "channel_delta" | "latent_attention"), mixer {sizes and constants
                      of that mixer}, mlp {"kind": "dense", "ff": n} or null (a layer without feed-forward)
  loop                {start, stop, times}: layers start..stop-1 run `times` times in a row with the same weights
                      (absent or null: every layer runs once)
Nothing here has a default that a model could silently rely on: a missing key is an error that names it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .model_config import ConfigError

MIXER_KEYS = {
    "lightning": ("heads", "dim", "vdim", "decay"),
    "channel_delta": ("heads", "kv_heads", "dim", "vdim", "conv"),
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot"),
}


def _need(d: dict, keys, where: str):
    missing = [k for k in keys if d.get(k) is None]
    if missing:
        raise ConfigError(f"config.json: {where} lacks {', '.join(missing)}")


@dataclass(frozen=True)
class NaditarLayer:
    type: str
    mixer: tuple                      # sorted (key, value) pairs; lists as tuples, "rot" as pairs of its own
    ff: Optional[int]                 # None: the layer has no feed-forward

    def m(self, key):
        return dict(self.mixer)[key]

    def mixer_dict(self) -> dict:
        d = dict(self.mixer)
        if "rot" in d:
            d["rot"] = dict(d["rot"])
        if "decay" in d:
            d["decay"] = list(d["decay"])
        return d


@dataclass(frozen=True)
class NaditarConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[NaditarLayer, ...]
    loop: Optional[Tuple[int, int, int]]          # (start, stop, times)
    max_position: int = 1 << 20                   # the design has no learned or tabulated positions: an engine limit only

    @classmethod
    def from_dict(cls, raw: dict) -> "NaditarConfig":
        _need(raw, ("vocab", "width", "layers", "norm"), "the top level")
        _need(raw["norm"], ("eps",), "'norm'")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            _need(entry, ("type", "mixer"), where)
            kind = entry["type"]
            if kind not in MIXER_KEYS:
                raise ConfigError(f"config.json: {where} has type '{kind}' (known: {', '.join(sorted(MIXER_KEYS))})")
            mx = dict(entry["mixer"])
            _need(mx, MIXER_KEYS[kind], f"{where}.mixer")
            if kind == "lightning":
                mx["decay"] = tuple(float(v) for v in mx["decay"])
                if len(mx["decay"]) != int(mx["heads"]):
                    raise ConfigError(f"config.json: {where}.mixer.decay has {len(mx['decay'])} entries for {mx['heads']} heads")
            if kind == "channel_delta":
                if int(mx["heads"]) % int(mx["kv_heads"]):
                    raise ConfigError(f"config.json: {where}: {mx['heads']} heads are not a multiple of {mx['kv_heads']} kv_heads")
                if int(mx["conv"]) < 1:
                    raise ConfigError(f"config.json: {where}.mixer.conv must be at least 1")
            if kind == "latent_attention":
                _need(mx["rot"], ("base", "dims"), f"{where}.mixer.rot")
                rot = {"base": float(mx["rot"]["base"]), "dims": int(mx["rot"]["dims"])}
                if rot["dims"] % 2 or rot["dims"] > int(mx["rot_dim"]):
                    raise ConfigError(f"config.json: {where}.mixer.rot.dims must be even and at most rot_dim")
                mx["rot"] = tuple(sorted(rot.items()))
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                _need(mlp, ("kind", "ff"), f"{where}.mlp")
                if mlp["kind"] != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind '{mlp['kind']}' is not supported (dense)")
                ff = int(mlp["ff"])
            layers.append(NaditarLayer(kind, tuple(sorted(mx.items())), ff))
        loop = raw.get("loop")
        if loop is not None:
            _need(loop, ("start", "stop", "times"), "'loop'")
            loop = (int(loop["start"]), int(loop["stop"]), int(loop["times"]))
            if not (0 <= loop[0] < loop[1] <= len(layers)) or loop[2] < 1:
                raise ConfigError(f"config.json: loop {loop} does not name a span of the {len(layers)} layers run at least once")
        return cls(architecture=raw.get("architecture") or (raw.get("architectures") or ["Naditar"])[0],
                   vocab=int(raw["vocab"]), width=int(raw["width"]), norm_eps=float(raw["norm"]["eps"]),
                   layers=tuple(layers), loop=loop, max_position=int(raw.get("max_position", 1 << 20)))

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": [{"type": layer.type, "mixer": layer.mixer_dict(),
                           "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff}} for layer in self.layers]}
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return out

    def describe(self) -> dict:
        return {"architecture": self.architecture, "layers": [layer.type for layer in self.layers], "loop": self.loop}
