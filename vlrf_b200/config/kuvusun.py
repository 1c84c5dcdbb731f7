"""Kuvusun's configuration: a decoder whose layers are listed one by one in config.json.

    {"architecture": "Kuvusun", "vocab": …, "width": …, "norm": {"eps": …, "groups": …},
     "layers": [{"type": "latent_attention" | "latent_attention_2", "mixer": {…}, "mlp": {…} | null}, …]}

Every layer names its mixer's kind and sizes and its feed-forward; nothing is shared between layers but the model's
width and norm.  A mixer of kind "latent_attention" makes its queries through a latent (`q_rank`) and has no rotated
part; "latent_attention_2" projects queries directly, has a rotated part (`rot_dim`, rotation `rot`: base and dims), a
gate on the merged heads, and may read an earlier layer's cache (`kv_from`).  A feed-forward is "dense" (`ff`) or
"moe" (`expert.ff`, `router.experts`, `router.top`, optionally `shared.ff`).
"""
from __future__ import annotations

import dataclasses

from .base import ConfigError, ModelConfig, key

MIXER_TYPES = ("latent_attention", "latent_attention_2")
MLP_KINDS = ("dense", "moe")


def _need(d: dict, name: str, kind, where: str):
    if not isinstance(d, dict) or name not in d:
        raise ConfigError(f"config.json: {where} lacks '{name}'")
    v = d[name]
    if kind is int:
        if isinstance(v, bool) or not (isinstance(v, int) or (isinstance(v, float) and v.is_integer())):
            raise ConfigError(f"config.json: {where}.{name} must be an integer, got {v!r}")
        return int(v)
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: {where}.{name} must be a number, got {v!r}")
        return float(v)
    return v


@dataclasses.dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float
    q_rank: int | None = None        # queries through a latent of this size (None: projected directly)
    rot_dim: int = 0                 # rotated query/key dimensions (0: none)
    rot_base: float = 0.0
    rot_dims: int = 0
    gated: bool = False              # sigmoid gate on the merged heads
    kv_from: int | None = None       # the layer whose cache this one reads (None: its own)


@dataclasses.dataclass(frozen=True)
class MlpConfig:
    kind: str
    ff: int                          # dense: inner size; moe: an expert's inner size
    experts: int = 0
    top: int = 0
    shared_ff: int | None = None


@dataclasses.dataclass
class KuvusunConfig(ModelConfig):
    model_type = "Kuvusun"

    vocab: int = key()
    width: int = key()
    norm: dict = key()
    layers: list = key()

    def to_dict(self) -> dict:
        return {"architecture": self.model_type, "vocab": self.vocab, "width": self.width, "norm": self.norm,
                "layers": self.layers}

    def validate(self) -> None:
        self._positive("vocab", self.vocab)
        self._positive("width", self.width)
        self.norm_eps = _need(self.norm, "eps", float, "norm")
        self.norm_groups = _need(self.norm, "groups", int, "norm")
        if not self.norm_eps > 0.0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        if self.norm_groups < 1 or self.width % self.norm_groups != 0:
            raise ConfigError(f"width ({self.width}) cannot be cut into norm.groups = {self.norm_groups} equal parts")
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        self.mixers, self.mlps = [], []
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", str, where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type '{kind}' is not one of {', '.join(MIXER_TYPES)}")
            m = _need(layer, "mixer", dict, where)
            mw = where + ".mixer"
            fields = dict(heads=_need(m, "heads", int, mw), dim=_need(m, "dim", int, mw), vdim=_need(m, "vdim", int, mw),
                          kv_rank=_need(m, "kv_rank", int, mw), scale=_need(m, "scale", float, mw))
            if kind == "latent_attention":
                fields["q_rank"] = _need(m, "q_rank", int, mw)
            else:
                rot = _need(m, "rot", dict, mw)
                fields.update(rot_dim=_need(m, "rot_dim", int, mw), rot_base=_need(rot, "base", float, mw + ".rot"),
                              rot_dims=_need(rot, "dims", int, mw + ".rot"), gated=True)
                if m.get("kv_from") is not None:
                    fields["kv_from"] = _need(m, "kv_from", int, mw)
            mc = LatentMixerConfig(**fields)
            for name in ("heads", "dim", "vdim", "kv_rank"):
                if getattr(mc, name) <= 0:
                    raise ConfigError(f"config.json: {mw}.{name} must be positive")
            if mc.q_rank is not None and mc.q_rank <= 0:
                raise ConfigError(f"config.json: {mw}.q_rank must be positive")
            if kind == "latent_attention_2":
                if mc.rot_dim <= 0 or mc.rot_dims <= 0 or mc.rot_dims % 2 != 0 or mc.rot_dims > mc.rot_dim or not mc.rot_base > 0:
                    raise ConfigError(f"config.json: {mw}: rot.dims ({mc.rot_dims}) must be even, positive and at most "
                                      f"rot_dim ({mc.rot_dim}), and rot.base positive")
            if mc.kv_from is not None:
                j = mc.kv_from
                if not (0 <= j < i) or self.mixers[j].kv_from is not None:
                    raise ConfigError(f"config.json: {mw}.kv_from = {j} must name an earlier layer with a cache of its own")
                o = self.mixers[j]
                if (o.kv_rank, o.rot_dim, o.rot_base, o.rot_dims) != (mc.kv_rank, mc.rot_dim, mc.rot_base, mc.rot_dims):
                    raise ConfigError(f"config.json: {mw}: kv_rank, rot_dim and rot differ from those of layer {j}, whose "
                                      f"cache it reads")
            self.mixers.append(mc)
            ml = layer.get("mlp")
            if ml is None:
                self.mlps.append(None)
                continue
            lw = where + ".mlp"
            mk = _need(ml, "kind", str, lw)
            if mk not in MLP_KINDS:
                raise ConfigError(f"config.json: {lw}.kind '{mk}' is not one of {', '.join(MLP_KINDS)}")
            if mk == "dense":
                cfg = MlpConfig("dense", _need(ml, "ff", int, lw))
            else:
                router = _need(ml, "router", dict, lw)
                shared = ml.get("shared")
                cfg = MlpConfig("moe", _need(_need(ml, "expert", dict, lw), "ff", int, lw + ".expert"),
                                experts=_need(router, "experts", int, lw + ".router"), top=_need(router, "top", int, lw + ".router"),
                                shared_ff=_need(shared, "ff", int, lw + ".shared") if shared is not None else None)
                if cfg.experts <= 0 or not (0 < cfg.top <= cfg.experts):
                    raise ConfigError(f"config.json: {lw}.router: top ({cfg.top}) must lie in 1…experts ({cfg.experts})")
                if cfg.shared_ff is not None and cfg.shared_ff <= 0:
                    raise ConfigError(f"config.json: {lw}.shared.ff must be positive")
            if cfg.ff <= 0:
                raise ConfigError(f"config.json: {lw}: the inner size must be positive")
            self.mlps.append(cfg)

    @property
    def n_layer(self) -> int:
        return len(self.layers)
