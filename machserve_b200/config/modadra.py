"""The Modadra decoder: its config.json keys, typed and checked, and its model as data.

config.json names the design under `architecture` and gives `vocab`, `width`, `norm.eps`, `residual_mult` (1 if absent),
`logit_softcap` (none if absent), optionally `max_positions`, and the list `layers`.  Every layer is a pre-norm one,
x += m * mixer(norm1(x)) and then x += m * mlp(norm2(x)), with m = residual_mult; it names its mixer under `type` with that
mixer's sizes under `mixer`, and its feed-forward under `mlp` (null: the layer has none).

* type `parallel`: two mixers side by side that read the same rows, `mixer.left` and `mixer.right`; each output is
  normed over the width with a plain weight of its own, and the result is half their sum.
  - left, attention: heads, kv_heads (heads if absent), dim (query/key size per head), vdim (dim if absent), scale,
    rot {dims, base} (a rotation of the first dims coordinates of every head in halves; none if absent), mask {size}
    (a sliding window; every earlier key if absent).  The softmax has one added to its denominator; every head's
    output has a sigmoid gate.
  - right, gated delta rule: heads (value heads), kv_heads (query/key heads; heads if absent), dim, vdim (dim if
    absent), conv (taps of the short convolution).
* mlp {kind: "moe", expert {ff}, router {experts, top, scale (1 if absent), groups {count, keep} (one group if absent)}}:
  experts without a gate and with the exact GELU; scores by sigmoid, a correction that enters the choice only, groups.

Tensor names: embed, final.norm, head, and per layer i: l<i>.norm1, l<i>.norm2, l<i>.mix.left.*, l<i>.mix.right.*,
l<i>.mix.left.out, l<i>.mix.right.out, l<i>.mlp.*.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .base import ConfigError, JsonReader, ModelConfig, register_architecture
from .spec import LayerSpec, ModelSpec, RunSpec, part
from .venarax import _sub

DEFAULT_MAX_POSITIONS = 1 << 20  # the design has no table of positions; a runner's cache bounds the context


@dataclass(frozen=True)
class WindowAttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int  # 0: no rotation
    rot_base: float
    window: Optional[int]

    @classmethod
    def read(cls, r: JsonReader) -> "WindowAttentionSizes":
        heads = r.integer("heads")
        kv = r.integer("kv_heads", heads)
        if heads % kv:
            raise ConfigError(f"{r.where}: heads {heads} is not a multiple of kv_heads {kv}")
        dim = r.integer("dim")
        rot = _sub(r.raw, "rot", r.where, required=False)
        dims = rot.integer("dims", minimum=0) if rot else 0
        if dims % 2 or dims > dim:
            raise ConfigError(f"{r.where}.rot: dims {dims} must be even and at most dim {dim}")
        mask = _sub(r.raw, "mask", r.where, required=False)
        return cls(heads, kv, dim, r.integer("vdim", dim), r.number("scale"), dims, rot.number("base") if rot and dims else 1.0,
                   mask.integer("size") if mask else None)

    def to_json(self) -> Dict[str, Any]:
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.rot_dims:
            out["rot"] = {"dims": self.rot_dims, "base": self.rot_base}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        return out


@dataclass(frozen=True)
class DeltaRuleSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def read(cls, r: JsonReader) -> "DeltaRuleSizes":
        heads = r.integer("heads")
        kv = r.integer("kv_heads", heads)
        if heads % kv:
            raise ConfigError(f"{r.where}: heads {heads} is not a multiple of kv_heads {kv}")
        dim = r.integer("dim")
        return cls(heads, kv, dim, r.integer("vdim", dim), r.integer("conv"))

    def to_json(self) -> Dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}


@dataclass(frozen=True)
class ParallelMixerSizes:
    left: WindowAttentionSizes
    right: DeltaRuleSizes

    @classmethod
    def read(cls, r: JsonReader) -> "ParallelMixerSizes":
        return cls(WindowAttentionSizes.read(_sub(r.raw, "left", r.where)), DeltaRuleSizes.read(_sub(r.raw, "right", r.where)))

    def to_json(self) -> Dict[str, Any]:
        return {"left": self.left.to_json(), "right": self.right.to_json()}


_MIXERS = {"parallel": ParallelMixerSizes}


@dataclass(frozen=True)
class GroupedMoeSizes:
    ff: int
    experts: int
    top: int
    scale: float
    groups: int
    keep: int

    @classmethod
    def read(cls, mlp: JsonReader) -> "GroupedMoeSizes":
        kind = mlp.string("kind")
        if kind != "moe":
            raise ConfigError(f"{mlp.where}: kind '{kind}' is not supported (moe)")
        expert, router = _sub(mlp.raw, "expert", mlp.where), _sub(mlp.raw, "router", mlp.where)
        experts, top = router.integer("experts"), router.integer("top")
        groups = _sub(router.raw, "groups", router.where, required=False)
        count, keep = (groups.integer("count"), groups.integer("keep")) if groups else (1, 1)
        if experts % count or keep > count:
            raise ConfigError(f"{router.where}: {experts} experts do not make {count} equal groups of which {keep} are kept")
        if top > experts // count * keep:
            raise ConfigError(f"{router.where}: top {top} is more than the {experts // count * keep} experts of the {keep} kept groups")
        return cls(expert.integer("ff"), experts, top, router.number("scale", 1.0), count, keep)

    def to_json(self) -> Dict[str, Any]:
        return {"kind": "moe", "expert": {"ff": self.ff},
                "router": {"experts": self.experts, "top": self.top, "scale": self.scale, "groups": {"count": self.groups, "keep": self.keep}}}


@dataclass(frozen=True)
class ModadraLayer:
    type: str
    mixer: Any  # ParallelMixerSizes
    mlp: Optional[GroupedMoeSizes]


@register_architecture("Modadra")
@dataclass(frozen=True)
class ModadraConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    residual_mult: float
    logit_softcap: Optional[float]
    max_positions: int
    layers: Tuple[ModadraLayer, ...]

    @classmethod
    def from_json(cls, raw: Mapping[str, Any]) -> "ModadraConfig":
        r = JsonReader(raw)
        norm = _sub(raw, "norm", "config.json")
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(listed):
            where = f"config.json.layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"{where}: must be an object")
            kind = JsonReader(entry, where).string("type")
            if kind not in _MIXERS:
                raise ConfigError(f"{where}: type '{kind}' is not a mixer of this design ({', '.join(sorted(_MIXERS))})")
            mlp = _sub(entry, "mlp", where, required=False)
            layers.append(ModadraLayer(kind, _MIXERS[kind].read(_sub(entry, "mixer", where)), GroupedMoeSizes.read(mlp) if mlp else None))
        cap = r.number("logit_softcap") if raw.get("logit_softcap") is not None else None
        return cls(r.integer("vocab"), r.integer("width"), norm.number("eps"), r.number("residual_mult", 1.0), cap,
                   r.integer("max_positions", DEFAULT_MAX_POSITIONS), tuple(layers))

    def to_json(self) -> Dict[str, Any]:
        out = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
            "residual_mult": self.residual_mult,
            "layers": [{"type": l.type, "mixer": l.mixer.to_json(), "mlp": l.mlp.to_json() if l.mlp else None} for l in self.layers],
        }
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    # ------------------------------------------------------------------ the model as data

    def _norm(self, name: str):
        return part("rmsnorm", tensor=name, size=self.width, eps=self.eps)

    def _mixer(self, layer: ModadraLayer, prefix: str):
        a, d = layer.mixer.left, layer.mixer.right
        position = None
        if a.rot_dims:
            position = part("rope", head_dim=a.dim, rotary_dim=a.rot_dims, theta=a.rot_base, pairing="half")
        left = part("rotary_gated_attention", prefix=prefix + "left.", hidden_size=self.width, num_heads=a.heads, num_kv_heads=a.kv_heads,
                    key_dim=a.dim, value_dim=a.vdim, scale=a.scale, window=a.window, sink=True, head_gate=True, position=position)
        right = part("gated_delta_rule", prefix=prefix + "right.", hidden_size=self.width, num_heads=d.heads, num_kv_heads=d.kv_heads,
                     key_dim=d.dim, value_dim=d.vdim, conv=d.conv, eps=self.eps)
        return part("two_mixers", left=left, right=right, left_norm=prefix + "left.out", right_norm=prefix + "right.out",
                    hidden_size=self.width, eps=self.eps, scale=0.5)

    def _mlp(self, layer: ModadraLayer, prefix: str):
        m = layer.mlp
        if m is None:
            return None
        return part("routed_experts", prefix=prefix, hidden_size=self.width, intermediate_size=m.ff, experts=m.experts, top=m.top,
                    activation="gelu", router_bias=False, gated=False, scoring="sigmoid", correction=True, groups=m.groups, keep=m.keep,
                    weight_scale=m.scale)

    def model_spec(self) -> ModelSpec:
        layers = []
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            mlp = self._mlp(layer, p + "mlp.")
            layers.append(LayerSpec(block="prenorm", mixer=self._mixer(layer, p + "mix."), feed_forward=mlp,
                                    mixer_norm=self._norm(p + "norm1"), feed_forward_norm=self._norm(p + "norm2") if mlp else None,
                                    prefix=p, block_params={"residual_scale": self.residual_mult}))
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            embedding=part("embedding", tensor="embed", vocab_size=self.vocab, hidden_size=self.width),
            layers=tuple(layers), run_order=tuple(RunSpec(i) for i in range(len(layers))), final_norm=self._norm("final.norm"),
            head=part("lm_head", tensor="head", tied_to=None, vocab_size=self.vocab, hidden_size=self.width, softcap=self.logit_softcap),
            max_positions=self.max_positions,
        )
