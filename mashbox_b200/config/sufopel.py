"""Typed configuration of the Sufopel decoder, read from config.json's own keys.

config.json: `architecture` (a string), `width`, `vocab`, `max_positions` (rows of the learned position table),
`embedding.scale`, `logit_scale`, `norm.eps`, `token_side.dim` (the per-layer token input; absent: none) and `layers`, a
list with one entry per layer: `type` ("latent_attention" or "channel_delta"), `mixer` (its sizes and constants) and
`mlp` ({"kind": "dense", "ff": F}, {"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top", "groups":
{"count", "keep"}}} or null).  Every layer has its own sizes; nothing is assumed equal between layers.

A latent_attention mixer: heads, dim, vdim, q_rank, kv_rank, scale, kv_from (the layer whose latents this one reads
instead of making its own).  A channel_delta mixer: heads, kv_heads, dim, vdim, conv (taps of the q/k/v convolutions;
absent: none).  The inner widths of its two low-rank products are not in config.json: the stored tensors have them
(`a_rank`, `g_rank` here are None then; random-weights mode sets them and writes them as keys of its own).
"""
from dataclasses import dataclass, field
from typing import Optional

from ..errors import ConfigError


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class DeltaMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: Optional[int] = None          # taps of the q/k/v convolutions; None: the mixer has none
    a_rank: Optional[int] = None        # inner width of the decay's low-rank product; None: as stored
    g_rank: Optional[int] = None        # inner width of the output gate's low-rank product; None: as stored


@dataclass(frozen=True)
class DenseFF:
    ff: int


@dataclass(frozen=True)
class RoutedFF:
    ff: int
    limit: float
    experts: int
    top: int
    groups: int = 1
    keep: int = 1


@dataclass(frozen=True)
class SufopelLayer:
    type: str
    mixer: object
    mlp: object                         # DenseFF, RoutedFF or None


@dataclass(frozen=True)
class SufopelConfig:
    architecture: str
    width: int
    vocab: int
    max_positions: int
    embedding_scale: float
    logit_scale: float
    norm_eps: float
    side_dim: Optional[int]
    layers: tuple
    extra: dict = field(default_factory=dict, compare=False, hash=False)

    @property
    def num_layers(self):
        return len(self.layers)

    @classmethod
    def from_hf(cls, cfg: dict) -> "SufopelConfig":
        arch = cfg.get("architecture") or (cfg.get("architectures") or [None])[0]

        def need(d, key, where):
            if not isinstance(d, dict) or d.get(key) is None:
                raise ConfigError(f"config.json has no `{where}{key}`")
            return d[key]

        layers = []
        for i, e in enumerate(need(cfg, "layers", "")):
            w = f"layers[{i}]."
            kind, m = need(e, "type", w), need(e, "mixer", w)
            w += "mixer."
            if kind == "latent_attention":
                kv_from = m.get("kv_from")
                mixer = LatentMixer(heads=int(need(m, "heads", w)), dim=int(need(m, "dim", w)), vdim=int(need(m, "vdim", w)),
                                    q_rank=int(need(m, "q_rank", w)), kv_rank=int(need(m, "kv_rank", w)),
                                    scale=float(m["scale"]) if m.get("scale") is not None else int(m["dim"]) ** -0.5,
                                    kv_from=int(kv_from) if kv_from is not None else None)
                if mixer.kv_from is not None:
                    j = mixer.kv_from
                    if not 0 <= j < i or layers[j].type != kind or layers[j].mixer.kv_from is not None:
                        raise ConfigError(f"config.json {w}kv_from = {j} must name an earlier latent_attention layer "
                                          f"with latents of its own")
                    if layers[j].mixer.kv_rank != mixer.kv_rank:
                        raise ConfigError(f"config.json {w}kv_from = {j}: that layer's latents have another size")
            elif kind == "channel_delta":
                heads = int(need(m, "heads", w))
                kv = int(m.get("kv_heads") or heads)
                if kv < 1 or heads % kv:
                    raise ConfigError(f"config.json {w}kv_heads = {kv} does not divide heads = {heads}")
                mixer = DeltaMixer(heads=heads, kv_heads=kv, dim=int(need(m, "dim", w)), vdim=int(need(m, "vdim", w)),
                                   conv=int(m["conv"]) if m.get("conv") else None,
                                   a_rank=int(m["a_rank"]) if m.get("a_rank") else None,
                                   g_rank=int(m["g_rank"]) if m.get("g_rank") else None)
            else:
                raise ConfigError(f"config.json layers[{i}].type = {kind!r} is not supported for {arch}")
            mlp, w = e.get("mlp"), f"layers[{i}].mlp."
            if mlp is None:
                ff = None
            elif mlp.get("kind", "dense") == "dense":
                ff = DenseFF(int(need(mlp, "ff", w)))
            elif mlp["kind"] == "moe":
                ex, r = need(mlp, "expert", w), need(mlp, "router", w)
                groups = r.get("groups") or {}
                ff = RoutedFF(ff=int(need(ex, "ff", w + "expert.")), limit=float(need(ex, "limit", w + "expert.")),
                              experts=int(need(r, "experts", w + "router.")), top=int(need(r, "top", w + "router.")),
                              groups=int(groups.get("count") or 1), keep=int(groups.get("keep") or groups.get("count") or 1))
                if ff.experts % ff.groups or not 1 <= ff.keep <= ff.groups or not 1 <= ff.top <= ff.keep * (ff.experts // ff.groups):
                    raise ConfigError(f"config.json {w}router: {ff.top} of {ff.experts} experts in {ff.groups} groups of "
                                      f"which {ff.keep} are kept cannot be chosen")
            else:
                raise ConfigError(f"config.json {w}kind = {mlp.get('kind')!r} is not supported for {arch}")
            layers.append(SufopelLayer(kind, mixer, ff))
        side = (cfg.get("token_side") or {}).get("dim")
        return cls(architecture=arch, width=int(need(cfg, "width", "")), vocab=int(need(cfg, "vocab", "")),
                   max_positions=int(need(cfg, "max_positions", "")),
                   embedding_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)),
                   logit_scale=float(cfg.get("logit_scale", 1.0)), norm_eps=float(need(cfg.get("norm"), "eps", "norm.")),
                   side_dim=int(side) if side else None, layers=tuple(layers),
                   extra={k: cfg[k] for k in ("bos_token_id", "eos_token_id") if k in cfg})

    def to_hf(self) -> dict:
        """The config.json that `from_hf` reads back to this configuration (random-weights mode writes it)."""
        out = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab,
               "max_positions": self.max_positions, "embedding": {"scale": self.embedding_scale},
               "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps}, "layers": []}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "latent_attention":
                e = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "q_rank": m.q_rank, "kv_rank": m.kv_rank,
                     "scale": m.scale}
                if m.kv_from is not None:
                    e["kv_from"] = m.kv_from
            else:
                e = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim}
                for key in ("conv", "a_rank", "g_rank"):
                    if getattr(m, key):
                        e[key] = getattr(m, key)
            f = layer.mlp
            if f is None:
                mlp = None
            elif isinstance(f, DenseFF):
                mlp = {"kind": "dense", "ff": f.ff}
            else:
                mlp = {"kind": "moe", "expert": {"ff": f.ff, "limit": f.limit},
                       "router": {"experts": f.experts, "top": f.top, "groups": {"count": f.groups, "keep": f.keep}}}
            out["layers"].append({"type": layer.type, "mixer": e, "mlp": mlp})
        out.update(self.extra)
        return out
