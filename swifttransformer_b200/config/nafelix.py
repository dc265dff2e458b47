"""Configuration of the Nafelix design: several residual streams, layers that pair a windowed attention whose heads
talk to one another with a gated delta rule, layers of gated windowed attention, dense and routed feed-forwards,
and a stretch of layers that may run several times.

``config.json`` is nested: ``layers`` is a list of objects, each with ``type`` ("parallel" or "attention"),
``mixer`` (its sizes and constants) and ``mlp`` (or null for none):

  parallel   ``mixer.left``  (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size``,
             ``rot.dims`` / ``rot.base``) and ``mixer.right`` (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv``)
  attention  ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size``, ``rot.dims`` / ``rot.base``
  mlp        ``kind`` "dense" with ``ff``; or "moe" with ``expert.ff``, ``expert.limit``, ``router.experts``,
             ``router.top``

Model-wide keys: ``vocab``, ``width``, ``streams``, ``norm.eps``, ``canon.taps`` and optionally
``loop.start / stop / times``.  The file names the design with the single string ``architecture``.  Every size and
constant is read from the file; an optional group the file does not mention switches its mechanism off (no
``mask``: every earlier key is seen; no ``rot``: nothing is rotated; no ``canon``: no input convolutions; no
``loop``: every layer runs once; no ``streams``: one residual stream).
"""
from __future__ import annotations

import copy
import dataclasses
from typing import Any, ClassVar, Dict, List, Optional, Tuple

from .base import ConfigError, ModelConfig, register_config


def _need(obj: Any, key: str, where: str, kinds=(int, float)) -> Any:
    if not isinstance(obj, dict) or key not in obj:
        raise ConfigError(f"Nafelix: config.json lacks '{where}{key}'")
    v = obj[key]
    if isinstance(v, bool) or not isinstance(v, kinds):
        raise ConfigError(f"Nafelix: '{where}{key}' has the wrong type ({v!r})")
    return v


def _positive_int(obj: Any, key: str, where: str) -> int:
    v = _need(obj, key, where, int)
    if v <= 0:
        raise ConfigError(f"Nafelix: '{where}{key}' must be a positive integer")
    return v


def _heads(mx: Any, where: str) -> None:
    for key in ("heads", "kv_heads", "dim", "vdim"):
        _positive_int(mx, key, where)
    if mx["heads"] % mx["kv_heads"]:
        raise ConfigError(f"Nafelix: '{where}heads' must be a multiple of '{where}kv_heads'")


def _attention(mx: Any, where: str) -> None:
    _heads(mx, where)
    _need(mx, "scale", where)
    if mx.get("mask") is not None:
        _positive_int(mx["mask"], "size", where + "mask.")
    if mx.get("rot") is not None:
        dims = _need(mx["rot"], "dims", where + "rot.", int)
        _need(mx["rot"], "base", where + "rot.")
        if dims < 0 or dims % 2 or dims > mx["dim"]:
            raise ConfigError(f"Nafelix: '{where}rot.dims' must be even and at most 'dim'")


@register_config
@dataclasses.dataclass(frozen=True)
class NafelixConfig(ModelConfig):
    ARCHITECTURE: ClassVar[str] = "Nafelix"

    vocab: int
    width: int
    layers: Tuple[Dict[str, Any], ...]
    norm_eps: float
    streams: int = 1
    canon_taps: int = 0                              # 0: no input convolutions
    loop: Optional[Tuple[int, int, int]] = None      # (start, stop, times)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "NafelixConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("Nafelix: config.json lacks 'layers' (a list with one object per layer)")
        loop = None
        if raw.get("loop"):
            lp = raw["loop"]
            loop = (_need(lp, "start", "loop.", int), _need(lp, "stop", "loop.", int), _need(lp, "times", "loop.", int))
        cfg = cls(vocab=_need(raw, "vocab", "", int), width=_need(raw, "width", "", int),
                  layers=tuple(copy.deepcopy(layers)), norm_eps=float(_need(raw.get("norm"), "eps", "norm.")),
                  streams=_need(raw, "streams", "", int) if raw.get("streams") is not None else 1,
                  canon_taps=_need(raw["canon"], "taps", "canon.", int) if raw.get("canon") else 0, loop=loop)
        cfg.validate()
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                               "streams": self.streams, "layers": copy.deepcopy(list(self.layers)),
                               "norm": {"eps": self.norm_eps}}
        if self.canon_taps:
            out["canon"] = {"taps": self.canon_taps}
        if self.loop:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return out

    def layer_runs(self) -> List[int]:
        """The layers in the order in which they run (a looped stretch appears ``times`` times in a row)."""
        n = len(self.layers)
        if not self.loop:
            return list(range(n))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("Nafelix: 'vocab' and 'width' must be positive")
        if self.norm_eps <= 0:
            raise ConfigError("Nafelix: 'norm.eps' must be positive")
        if not 1 <= self.streams <= 8:
            raise ConfigError("Nafelix: 'streams' must be between 1 and 8")
        if not 0 <= self.canon_taps <= 8:
            raise ConfigError("Nafelix: 'canon.taps' must be between 1 and 8")
        if self.loop is not None:
            start, stop, times = self.loop
            if not (0 <= start < stop <= len(self.layers)) or times < 1:
                raise ConfigError("Nafelix: 'loop' needs 0 <= start < stop <= number of layers and times >= 1")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            kind = layer.get("type") if isinstance(layer, dict) else None
            mx = layer.get("mixer") if isinstance(layer, dict) else None
            if kind == "parallel":
                _attention((mx or {}).get("left"), where + "mixer.left.")
                right = (mx or {}).get("right")
                _heads(right, where + "mixer.right.")
                _positive_int(right, "conv", where + "mixer.right.")
            elif kind == "attention":
                _attention(mx, where + "mixer.")
            else:
                raise ConfigError(f"Nafelix: '{where}type' = {kind!r} is not a known layer type (parallel, attention)")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if mlp.get("kind") == "dense":
                _positive_int(mlp, "ff", where + "mlp.")
            elif mlp.get("kind") == "moe":
                _positive_int(mlp.get("expert"), "ff", where + "mlp.expert.")
                _need(mlp.get("expert"), "limit", where + "mlp.expert.")
                n = _positive_int(mlp.get("router"), "experts", where + "mlp.router.")
                if _positive_int(mlp.get("router"), "top", where + "mlp.router.") > n:
                    raise ConfigError(f"Nafelix: '{where}mlp.router.top' exceeds the number of experts")
            else:
                raise ConfigError(f"Nafelix: '{where}mlp.kind' = {mlp.get('kind')!r} is not known (dense, moe)")
