"""Typed configuration of the Luzosun decoder, read from config.json's own keys.

config.json: `architecture` (a string), `width`, `vocab`, `embedding.scale`, `norm.eps`, `canon.taps` (the input
convolution of every layer's mixer; absent: none; 1 is a filter of one tap, which keeps no state) and `layers`, a list with one entry per layer: `type`
(the mixer kind; "attention" is the differential attention mixer), `mixer` (its sizes and constants) and `mlp`
({"kind": "dense", "ff": F} or null).  Every layer has its own sizes; nothing is assumed equal between layers.  A
mixer entry: heads, kv_heads, dim (per map), vdim, conv (taps of the q/k/v convolutions; absent: none), diff, scale, mask.size (the
block of positions a query sees; absent: all earlier keys), rot {base, dims, scaling.factor} (absent: no rotation),
kv_from (the layer whose keys and values this one reads instead of making its own).
"""
from dataclasses import dataclass, field
from typing import Optional

from ..errors import ConfigError


@dataclass(frozen=True)
class LuzosunMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    diff: float
    scale: float
    conv: Optional[int] = None         # taps of the q/k/v convolutions; None: the mixer has none
    mask_size: Optional[int] = None
    rot_base: Optional[float] = None
    rot_dims: int = 0
    rot_factor: Optional[float] = None
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class LuzosunLayer:
    type: str
    mixer: LuzosunMixer
    ff: Optional[int]                   # the dense feed-forward's inner width; None: the layer has none


@dataclass(frozen=True)
class LuzosunConfig:
    architecture: str
    width: int
    vocab: int
    embedding_scale: float
    norm_eps: float
    canon_taps: int
    layers: tuple
    extra: dict = field(default_factory=dict, compare=False, hash=False)

    @property
    def num_layers(self):
        return len(self.layers)

    @classmethod
    def from_hf(cls, cfg: dict) -> "LuzosunConfig":
        arch = cfg.get("architecture") or (cfg.get("architectures") or [None])[0]

        def need(d, key, where):
            if not isinstance(d, dict) or d.get(key) is None:
                raise ConfigError(f"config.json has no `{where}{key}`")
            return d[key]

        layers = []
        entries = need(cfg, "layers", "")
        for i, e in enumerate(entries):
            w = f"layers[{i}]."
            kind = need(e, "type", w)
            if kind != "attention":
                raise ConfigError(f"config.json {w}type = {kind!r} is not supported for {arch}")
            m = need(e, "mixer", w)
            w += "mixer."
            heads, kv = int(need(m, "heads", w)), int(m.get("kv_heads") or m["heads"])
            if kv < 1 or heads % kv:
                raise ConfigError(f"config.json {w}kv_heads = {kv} does not divide heads = {heads}")
            dim = int(need(m, "dim", w))
            rot = m.get("rot") or None
            rot_dims = int(need(rot, "dims", w + "rot.")) if rot else 0
            if rot and (rot_dims < 2 or rot_dims % 2 or rot_dims > dim):
                raise ConfigError(f"config.json {w}rot.dims = {rot_dims} must be even and at most dim = {dim}")
            kv_from = m.get("kv_from")
            if kv_from is not None:
                kv_from = int(kv_from)
                if not 0 <= kv_from < i or layers[kv_from].mixer.kv_from is not None:
                    raise ConfigError(f"config.json {w}kv_from = {kv_from} must name an earlier layer with keys and "
                                      f"values of its own")
                o = layers[kv_from].mixer
                if (o.kv_heads, o.dim, o.vdim) != (kv, dim, int(need(m, "vdim", w))):
                    raise ConfigError(f"config.json {w}kv_from = {kv_from}: that layer's keys and values have other sizes")
            mlp = e.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise ConfigError(f"config.json layers[{i}].mlp.kind = {mlp.get('kind')!r} is not supported for {arch}")
            mask = m.get("mask") or {}
            layers.append(LuzosunLayer(kind, LuzosunMixer(
                heads=heads, kv_heads=kv, dim=dim, vdim=int(need(m, "vdim", w)), diff=float(need(m, "diff", w)),
                scale=float(m["scale"]) if m.get("scale") is not None else dim ** -0.5,
                conv=int(m["conv"]) if m.get("conv") else None,
                mask_size=int(mask["size"]) if mask.get("size") else None,
                rot_base=float(need(rot, "base", w + "rot.")) if rot else None, rot_dims=rot_dims,
                rot_factor=float(rot["scaling"]["factor"]) if rot and (rot.get("scaling") or {}).get("factor") else None,
                kv_from=kv_from), int(need(mlp, "ff", f"layers[{i}].mlp.")) if mlp is not None else None))
        return cls(architecture=arch, width=int(need(cfg, "width", "")), vocab=int(need(cfg, "vocab", "")),
                   embedding_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)),
                   norm_eps=float(need(cfg.get("norm"), "eps", "norm.")),
                   canon_taps=int((cfg.get("canon") or {}).get("taps") or 0), layers=tuple(layers),
                   extra={k: cfg[k] for k in ("bos_token_id", "eos_token_id") if k in cfg})

    def to_hf(self) -> dict:
        """The config.json that `from_hf` reads back to this configuration (random-weights mode writes it)."""
        out = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab,
               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps}, "layers": []}
        if self.canon_taps:
            out["canon"] = {"taps": self.canon_taps}
        for layer in self.layers:
            m = layer.mixer
            e = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "diff": m.diff,
                 "scale": m.scale}
            if m.conv:
                e["conv"] = m.conv
            if m.mask_size:
                e["mask"] = {"size": m.mask_size}
            if m.rot_base is not None:
                e["rot"] = {"base": m.rot_base, "dims": m.rot_dims}
                if m.rot_factor:
                    e["rot"]["scaling"] = {"factor": m.rot_factor}
            if m.kv_from is not None:
                e["kv_from"] = m.kv_from
            out["layers"].append({"type": layer.type, "mixer": e,
                                  "mlp": {"kind": "dense", "ff": layer.ff} if layer.ff else None})
        out.update(self.extra)
        return out
