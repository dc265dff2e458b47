"""Configuration of the Norelix design: layers that pair a windowed attention with a gated delta rule, and layers
of gated attention that may share another layer's keys and values.

``config.json`` is nested: ``layers`` is a list of objects, each with ``type`` ("parallel" or "attention"),
``mixer`` (its sizes and constants) and ``mlp`` (``kind`` "dense" with ``ff`` and ``limit``; or null).

  parallel   ``mixer.left``  (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size`` /
             ``mask.keep_first``, ``rot.dims`` / ``rot.base``), ``mixer.right`` (``heads``, ``kv_heads``, ``dim``,
             ``vdim``, ``conv``), ``mixer.left_scale``, ``mixer.right_scale``
  attention  ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``q_temp.coef`` / ``q_temp.every``, and
             optionally ``kv_from``: the index of an earlier attention layer whose keys and values this one reads

Model-wide keys: ``vocab``, ``width``, ``norm.eps``.  The file names the design with the single string
``architecture``.  Every size and constant is read from the file; an optional group the file does not mention
switches its mechanism off (no ``mask``: every earlier key is seen; no ``rot``: nothing is rotated; no ``q_temp``:
no temperature).
"""
from __future__ import annotations

import copy
import dataclasses
from typing import Any, ClassVar, Dict, Tuple

from .base import ConfigError, ModelConfig, register_config


def _need(obj: Any, key: str, where: str, kinds=(int, float)) -> Any:
    if not isinstance(obj, dict) or key not in obj:
        raise ConfigError(f"Norelix: config.json lacks '{where}{key}'")
    v = obj[key]
    if isinstance(v, bool) or not isinstance(v, kinds):
        raise ConfigError(f"Norelix: '{where}{key}' has the wrong type ({v!r})")
    return v


def _positive_int(obj: Any, key: str, where: str) -> int:
    v = _need(obj, key, where, int)
    if v <= 0:
        raise ConfigError(f"Norelix: '{where}{key}' must be a positive integer")
    return v


def _heads(mx: Any, where: str) -> None:
    for key in ("heads", "kv_heads", "dim", "vdim"):
        _positive_int(mx, key, where)
    if mx["heads"] % mx["kv_heads"]:
        raise ConfigError(f"Norelix: '{where}heads' must be a multiple of '{where}kv_heads'")


@register_config
@dataclasses.dataclass(frozen=True)
class NorelixConfig(ModelConfig):
    ARCHITECTURE: ClassVar[str] = "Norelix"

    vocab: int
    width: int
    layers: Tuple[Dict[str, Any], ...]
    norm_eps: float

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "NorelixConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("Norelix: config.json lacks 'layers' (a list with one object per layer)")
        cfg = cls(vocab=_need(raw, "vocab", "", int), width=_need(raw, "width", "", int),
                  layers=tuple(copy.deepcopy(layers)), norm_eps=float(_need(raw.get("norm"), "eps", "norm.")))
        cfg.validate()
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps}}

    def kv_source(self, i: int) -> int:
        """The layer whose keys and values attention layer ``i`` reads (itself unless ``kv_from`` says otherwise)."""
        src = self.layers[i]["mixer"].get("kv_from")
        return i if src is None else int(src)

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("Norelix: 'vocab' and 'width' must be positive")
        if self.norm_eps <= 0:
            raise ConfigError("Norelix: 'norm.eps' must be positive")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            kind = layer.get("type") if isinstance(layer, dict) else None
            mx = layer.get("mixer") if isinstance(layer, dict) else None
            if kind == "parallel":
                left, right = (mx or {}).get("left"), (mx or {}).get("right")
                _heads(left, where + "mixer.left.")
                _need(left, "scale", where + "mixer.left.")
                if left.get("mask") is not None:
                    _positive_int(left["mask"], "size", where + "mixer.left.mask.")
                    if left["mask"].get("keep_first") is not None and _need(left["mask"], "keep_first",
                                                                              where + "mixer.left.mask.", int) < 0:
                        raise ConfigError(f"Norelix: '{where}mixer.left.mask.keep_first' must not be negative")
                if left.get("rot") is not None:
                    dims = _need(left["rot"], "dims", where + "mixer.left.rot.", int)
                    _need(left["rot"], "base", where + "mixer.left.rot.")
                    if dims < 0 or dims % 2 or dims > left["dim"]:
                        raise ConfigError(f"Norelix: '{where}mixer.left.rot.dims' must be even and at most 'dim'")
                _heads(right, where + "mixer.right.")
                _positive_int(right, "conv", where + "mixer.right.")
                for key in ("left_scale", "right_scale"):
                    if mx.get(key) is not None:
                        _need(mx, key, where + "mixer.")
            elif kind == "attention":
                _heads(mx, where + "mixer.")
                _need(mx, "scale", where + "mixer.")
                if mx.get("q_temp") is not None:
                    _need(mx["q_temp"], "coef", where + "mixer.q_temp.")
                    _positive_int(mx["q_temp"], "every", where + "mixer.q_temp.")
                if mx.get("kv_from") is not None:
                    j = _need(mx, "kv_from", where + "mixer.", int)
                    src = self.layers[j] if 0 <= j < i else None
                    if src is None or src.get("type") != "attention" or src["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"Norelix: '{where}mixer.kv_from' must name an earlier attention layer "
                                          f"with keys and values of its own")
                    if any(src["mixer"].get(k) != mx[k] for k in ("kv_heads", "dim", "vdim")):
                        raise ConfigError(f"Norelix: '{where}mixer.kv_from': the two layers differ in 'kv_heads', "
                                          f"'dim' or 'vdim'")
            else:
                raise ConfigError(f"Norelix: '{where}type' = {kind!r} is not a known layer type (parallel, attention)")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if mlp.get("kind") != "dense":
                raise ConfigError(f"Norelix: '{where}mlp.kind' = {mlp.get('kind')!r} is not known (dense)")
            _positive_int(mlp, "ff", where + "mlp.")
            _need(mlp, "limit", where + "mlp.")
