"""Typed configuration of the Namesun design, read from its own config.json keys.

config.json names every size and every constant that differs between models of the design:
  architecture        "Namesun"
  vocab, width        vocabulary and width of the residual stream
  norm.eps            the one epsilon of all root-mean-square norms (also the unit norms inside the mixers)
  residual_mult       the number every sublayer's normed output is multiplied by before it joins the stream
  layers[i]           type ("attention" | "retention"), mixer {sizes and constants of that mixer}, and
                      mlp: null (no feed-forward), {"kind": "dense", "ff": n}, or {"kind": "moe", "router": {experts, top,
                      groups: {count, keep} (optional)}, "expert": {ff, limit}, "shared": {ff, limit} (optional)}
    attention mixer   heads, kv_heads, dim (query/key size per head), vdim, scale, mask {size} (optional: blocks of
                      positions that do not see each other), v_mix (optional: blend the values of the first such layer in)
    retention mixer   heads, dim, vdim, decay [one per head], rot {dims, base}
A missing key is an error that names it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .model_config import ConfigError

MIXER_KEYS = {
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale"),
    "retention": ("heads", "dim", "vdim", "decay", "rot"),
}


def _need(d, keys, where: str):
    if not isinstance(d, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    missing = [k for k in keys if d.get(k) is None]
    if missing:
        raise ConfigError(f"config.json: {where} lacks {', '.join(missing)}")


@dataclass(frozen=True)
class NamesunMLP:
    kind: str                                     # "dense" | "moe"
    ff: int                                       # dense: the intermediate size; moe: an expert's
    experts: int = 0
    top: int = 0
    groups: Optional[Tuple[int, int]] = None      # (count, keep)
    limit: float = 0.0
    shared: Optional[Tuple[int, float]] = None    # (ff, limit) of the expert that every token uses

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        router = {"experts": self.experts, "top": self.top}
        if self.groups is not None:
            router["groups"] = {"count": self.groups[0], "keep": self.groups[1]}
        out = {"kind": "moe", "router": router, "expert": {"ff": self.ff, "limit": self.limit}}
        if self.shared is not None:
            out["shared"] = {"ff": self.shared[0], "limit": self.shared[1]}
        return out


@dataclass(frozen=True)
class NamesunLayer:
    type: str
    mixer: tuple                                  # sorted (key, value) pairs; lists as tuples, nested objects as pairs
    mlp: Optional[NamesunMLP]

    def mixer_dict(self) -> dict:
        d = dict(self.mixer)
        for key in ("rot", "mask"):
            if d.get(key) is not None:
                d[key] = dict(d[key])
        if "decay" in d:
            d["decay"] = list(d["decay"])
        return d


def _read_mlp(mlp, where: str) -> Optional[NamesunMLP]:
    if mlp is None:
        return None
    _need(mlp, ("kind",), where)
    if mlp["kind"] == "dense":
        _need(mlp, ("ff",), where)
        return NamesunMLP("dense", int(mlp["ff"]))
    if mlp["kind"] != "moe":
        raise ConfigError(f"config.json: {where}.kind '{mlp['kind']}' is not one of dense, moe")
    _need(mlp, ("router", "expert"), where)
    _need(mlp["router"], ("experts", "top"), f"{where}.router")
    _need(mlp["expert"], ("ff", "limit"), f"{where}.expert")
    experts, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    groups = mlp["router"].get("groups")
    if groups is not None:
        _need(groups, ("count", "keep"), f"{where}.router.groups")
        groups = (int(groups["count"]), int(groups["keep"]))
        if groups[0] < 1 or experts % groups[0] or not 1 <= groups[1] <= groups[0]:
            raise ConfigError(f"config.json: {where}.router.groups {groups} do not cut {experts} experts into equal groups of which some are kept")
    allowed = experts if groups is None else experts // groups[0] * groups[1]
    if not 1 <= top <= allowed:
        raise ConfigError(f"config.json: {where}.router.top is {top}; {allowed} experts can be chosen")
    shared = mlp.get("shared")
    if shared is not None:
        _need(shared, ("ff", "limit"), f"{where}.shared")
        shared = (int(shared["ff"]), float(shared["limit"]))
    return NamesunMLP("moe", int(mlp["expert"]["ff"]), experts, top, groups, float(mlp["expert"]["limit"]), shared)


@dataclass(frozen=True)
class NamesunConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    layers: Tuple[NamesunLayer, ...]
    max_position: int = 1 << 20                   # the design tabulates no positions: an engine limit only

    @classmethod
    def from_dict(cls, raw: dict) -> "NamesunConfig":
        _need(raw, ("vocab", "width", "layers", "norm", "residual_mult"), "the top level")
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
            if kind == "attention":
                if int(mx["heads"]) % int(mx["kv_heads"]):
                    raise ConfigError(f"config.json: {where}: {mx['heads']} heads are not a multiple of {mx['kv_heads']} kv_heads")
                mask = mx.get("mask")
                if mask is not None:
                    _need(mask, ("size",), f"{where}.mixer.mask")
                    if int(mask["size"]) < 1:
                        raise ConfigError(f"config.json: {where}.mixer.mask.size must be at least 1")
                    mask = (("size", int(mask["size"])),)
                mx["mask"] = mask
                mx["v_mix"] = bool(mx.get("v_mix", False))
                mx["scale"] = float(mx["scale"])
            else:
                mx["decay"] = tuple(float(v) for v in mx["decay"])
                if len(mx["decay"]) != int(mx["heads"]):
                    raise ConfigError(f"config.json: {where}.mixer.decay has {len(mx['decay'])} entries for {mx['heads']} heads")
                _need(mx["rot"], ("base", "dims"), f"{where}.mixer.rot")
                rot = {"base": float(mx["rot"]["base"]), "dims": int(mx["rot"]["dims"])}
                if rot["dims"] % 2 or not 0 <= rot["dims"] <= int(mx["dim"]):
                    raise ConfigError(f"config.json: {where}.mixer.rot.dims must be even and at most dim")
                mx["rot"] = tuple(sorted(rot.items()))
            layers.append(NamesunLayer(kind, tuple(sorted(mx.items())), _read_mlp(entry.get("mlp"), f"{where}.mlp")))
        return cls(architecture=raw.get("architecture") or (raw.get("architectures") or ["Namesun"])[0],
                   vocab=int(raw["vocab"]), width=int(raw["width"]), norm_eps=float(raw["norm"]["eps"]),
                   residual_mult=float(raw["residual_mult"]), layers=tuple(layers),
                   max_position=int(raw.get("max_position", 1 << 20)))

    def to_dict(self) -> dict:
        layers = []
        for layer in self.layers:
            m = layer.mixer_dict()
            if layer.type == "attention":
                if m.get("mask") is None:
                    m.pop("mask", None)
                if not m.get("v_mix"):
                    m.pop("v_mix", None)
            layers.append({"type": layer.type, "mixer": m, "mlp": None if layer.mlp is None else layer.mlp.to_dict()})
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "residual_mult": self.residual_mult, "layers": layers}

    def describe(self) -> dict:
        return {"architecture": self.architecture,
                "layers": [f"{layer.type}+{layer.mlp.kind if layer.mlp else 'none'}" for layer in self.layers]}
