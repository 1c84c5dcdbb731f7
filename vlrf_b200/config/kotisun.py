"""Kotisun's configuration: a decoder whose layers are listed one by one in config.json.

    {"architecture": "Kotisun", "vocab": …, "width": …, "norm": {"eps": …}, "embedding": {"scale": …},
     "streams": …, "loop": {"start": …, "stop": …, "times": …}, "logit_softcap": …,
     "layers": [{"type": "parallel", "mixer": {"left": {…}, "right": {…}, "left_scale": …, "right_scale": …},
                 "mlp": {"kind": "dense", "ff": …} | null}, …]}

A layer of type "parallel" runs two mixers on the same input.  `left` is softmax attention: `heads`, `kv_heads`, `dim`
(queries and keys), `vdim` (values), `scale`, optionally `mask.size` (a sliding window) and `rot` (`base`, `dims`,
optionally `scaling.factor`).  `right` is a state-space recurrence: `heads`, `vdim`, `state`, `groups`, `conv` (taps),
`norm_groups`.  `streams`: the residual is carried in that many rows per token (absent: the plain residual sum).
`loop`: layers start … stop − 1 run `times` times in a row with the same weights, each pass with a cache and state of
its own.  Every size and constant is per layer; nothing but width, norm.eps and streams is shared.
"""
from __future__ import annotations

import dataclasses

from .base import ConfigError, ModelConfig, key
from .kuvusun import _need

LAYER_TYPES = ("parallel",)
MLP_KINDS = ("dense",)


@dataclasses.dataclass(frozen=True)
class AttentionBranchConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int = 0                  # 0: every earlier key is visible
    rot_dims: int = 0                # rotated entries of a head (0: none)
    rot_base: float = 0.0
    rot_factor: float = 1.0          # linear scaling: every frequency is divided by it


@dataclasses.dataclass(frozen=True)
class RecurrentBranchConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclasses.dataclass(frozen=True)
class ParallelLayerConfig:
    left: AttentionBranchConfig
    right: RecurrentBranchConfig
    left_scale: float
    right_scale: float
    ff: int | None                   # inner size of the gated feed-forward, or None for a layer without one


def _optional(d: dict, name: str):
    v = d.get(name) if isinstance(d, dict) else None
    return v if isinstance(v, dict) else None


@dataclasses.dataclass
class KotisunConfig(ModelConfig):
    model_type = "Kotisun"

    vocab: int = key()
    width: int = key()
    norm: dict = key()
    layers: list = key()
    embedding: dict = key(default=None, nullable=True)
    streams: int = key(default=None, nullable=True)
    loop: dict = key(default=None, nullable=True)
    logit_softcap: float = key(default=None, nullable=True)

    def to_dict(self) -> dict:
        out = {"architecture": self.model_type, "vocab": self.vocab, "width": self.width, "norm": self.norm, "layers": self.layers}
        for name in ("embedding", "streams", "loop", "logit_softcap"):
            if getattr(self, name) is not None:
                out[name] = getattr(self, name)
        return out

    def validate(self) -> None:
        self._positive("vocab", self.vocab)
        self._positive("width", self.width)
        self.norm_eps = _need(self.norm, "eps", float, "norm")
        if not self.norm_eps > 0.0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        self.embedding_scale = _need(self.embedding, "scale", float, "embedding") if self.embedding is not None else 1.0
        if self.streams is not None and not (1 <= self.streams <= 16):
            raise ConfigError(f"streams ({self.streams}) must lie in 1…16")
        if self.logit_softcap is not None and not self.logit_softcap > 0.0:
            raise ConfigError(f"logit_softcap must be positive, got {self.logit_softcap}")
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        self.layer_configs = [self._layer(i, layer) for i, layer in enumerate(self.layers)]
        n = len(self.layers)
        self.layer_order = list(range(n))
        if self.loop is not None:
            a, b, k = (_need(self.loop, name, int, "loop") for name in ("start", "stop", "times"))
            if not (0 <= a <= b <= n) or k < 1:
                raise ConfigError(f"loop: start {a}, stop {b}, times {k} do not name a range of the {n} layers run at least once")
            self.layer_order = list(range(a)) + list(range(a, b)) * k + list(range(b, n))

    def _layer(self, i: int, layer) -> ParallelLayerConfig:
        where = f"layers[{i}]"
        kind = _need(layer, "type", str, where)
        if kind not in LAYER_TYPES:
            raise ConfigError(f"config.json: {where}.type '{kind}' is not one of {', '.join(LAYER_TYPES)}")
        m = _need(layer, "mixer", dict, where)
        lw, rw = where + ".mixer.left", where + ".mixer.right"
        lf, rt = _need(m, "left", dict, where + ".mixer"), _need(m, "right", dict, where + ".mixer")
        fields = dict(heads=_need(lf, "heads", int, lw), kv_heads=_need(lf, "kv_heads", int, lw), dim=_need(lf, "dim", int, lw),
                      vdim=_need(lf, "vdim", int, lw), scale=_need(lf, "scale", float, lw))
        mask = _optional(lf, "mask")
        if mask is not None:
            fields["window"] = _need(mask, "size", int, lw + ".mask")
            if fields["window"] <= 0:
                raise ConfigError(f"config.json: {lw}.mask.size must be positive")
        rot = _optional(lf, "rot")
        if rot is not None:
            fields.update(rot_dims=_need(rot, "dims", int, lw + ".rot"), rot_base=_need(rot, "base", float, lw + ".rot"))
            scaling = _optional(rot, "scaling")
            if scaling is not None:
                fields["rot_factor"] = _need(scaling, "factor", float, lw + ".rot.scaling")
        left = AttentionBranchConfig(**fields)
        if min(left.heads, left.kv_heads, left.dim, left.vdim) <= 0 or left.heads % left.kv_heads != 0:
            raise ConfigError(f"config.json: {lw}: sizes must be positive and heads ({left.heads}) a multiple of kv_heads ({left.kv_heads})")
        if rot is not None and (left.rot_dims <= 0 or left.rot_dims % 2 != 0 or left.rot_dims > left.dim or not left.rot_base > 0
                                or not left.rot_factor > 0):
            raise ConfigError(f"config.json: {lw}.rot: dims ({left.rot_dims}) must be even, positive and at most dim ({left.dim}); "
                              f"base and scaling.factor positive")
        right = RecurrentBranchConfig(heads=_need(rt, "heads", int, rw), vdim=_need(rt, "vdim", int, rw), state=_need(rt, "state", int, rw),
                                      groups=_need(rt, "groups", int, rw), conv=_need(rt, "conv", int, rw),
                                      norm_groups=_need(rt, "norm_groups", int, rw))
        if min(right.heads, right.vdim, right.state, right.groups, right.conv, right.norm_groups) <= 0 or right.heads % right.groups != 0 \
                or (right.heads * right.vdim) % right.norm_groups != 0:
            raise ConfigError(f"config.json: {rw}: sizes must be positive, heads a multiple of groups, and heads·vdim of norm_groups")
        ml = layer.get("mlp")
        ff = None
        if ml is not None:
            mk = _need(ml, "kind", str, where + ".mlp")
            if mk not in MLP_KINDS:
                raise ConfigError(f"config.json: {where}.mlp.kind '{mk}' is not one of {', '.join(MLP_KINDS)}")
            ff = _need(ml, "ff", int, where + ".mlp")
            if ff <= 0:
                raise ConfigError(f"config.json: {where}.mlp.ff must be positive")
        return ParallelLayerConfig(left, right, _need(m, "left_scale", float, where + ".mixer"),
                                   _need(m, "right_scale", float, where + ".mixer"), ff)

    @property
    def n_layer(self) -> int:
        return len(self.layers)
