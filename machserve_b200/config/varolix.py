"""The Varolix decoder: its config.json keys, typed and checked, and its model as data.

config.json names the design under `architecture` and gives `vocab`, `width`, `norm.eps`, the list `layers` and, optionally,
`loop`.  Every layer is a pre-norm one, x += mixer(norm1(x)) and then x += mlp(norm2(x)); it names its mixer under `type`
with that mixer's sizes under `mixer`, and its feed-forward under `mlp` (null: the layer has none).

* type `attention`: heads, kv_heads (heads if absent), dim (query/key size per head), vdim (dim if absent), scale,
  rot {dims, base, scaling {factor, original, fast, slow} (none if absent)}: grouped heads with biases on q, k and v, a
  rotation in halves of the first rot.dims coordinates of every head, optionally stretched for long contexts; causal softmax.
* type `parallel`: two mixers side by side that read the same rows, `mixer.left` and `mixer.right`; the result is
  left_scale * left + right_scale * right.
  - left, attention: heads, kv_heads, dim, vdim, scale, q_temp {coef, every} (none if absent).  Biases on q, k, v and the
    output; every q and k head normed with a weight the heads share; no rotation; a query temperature by position.
  - right, matrix memory: heads, dim, vdim (dim if absent), gate_cap.
* type `latent_attention`: heads, dim (unrotated) and rot_dim (rotated query/key sizes per head), vdim, kv_rank (the cached
  latent), q_rank (the queries' latent), scale, rot {dims, base}.  A sink per head in the softmax, a gate per head.
* mlp {kind: "dense", ff}: W_down (gelu_tanh(W_gate h) * (W_up h)).

`loop` {start, stop, times}: layers start..stop-1 run `times` times in a row with the same weights; every pass has a cache
or state of its own, and nothing else happens between passes.  The config gives no limit on positions: the engine's own
limit (its cache) stands.

Tensor names: embed, final.norm, head, and per layer i: l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.{gate,up,down}.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .base import ConfigError, JsonReader, ModelConfig, register_architecture
from .spec import LayerSpec, ModelSpec, RunSpec, part
from .venarax import NO_POSITION_LIMIT, LayerLoop, _sub


def _heads(r: JsonReader) -> Tuple[int, int]:
    heads = r.integer("heads")
    kv = r.integer("kv_heads", heads)
    if heads % kv:
        raise ConfigError(f"{r.where}: heads {heads} is not a multiple of kv_heads {kv}")
    return heads, kv


@dataclass(frozen=True)
class RotaryScaling:
    factor: float
    original: float
    fast: float
    slow: float

    def to_json(self) -> Dict[str, Any]:
        return {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}


@dataclass(frozen=True)
class RotaryAttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int  # 0: no rotation
    rot_base: float
    scaling: Optional[RotaryScaling]

    @classmethod
    def read(cls, r: JsonReader) -> "RotaryAttentionSizes":
        heads, kv = _heads(r)
        dim = r.integer("dim")
        rot = _sub(r.raw, "rot", r.where, required=False)
        dims = rot.integer("dims", minimum=0) if rot else 0
        if dims % 2 or dims > dim:
            raise ConfigError(f"{r.where}.rot: dims {dims} must be even and at most dim {dim}")
        scaling = _sub(rot.raw, "scaling", rot.where, required=False) if rot and dims else None
        if scaling is not None:
            scaling = RotaryScaling(scaling.number("factor"), scaling.number("original"), scaling.number("fast"), scaling.number("slow"))
        return cls(heads, kv, dim, r.integer("vdim", dim), r.number("scale"), dims, rot.number("base") if rot and dims else 1.0, scaling)

    def to_json(self) -> Dict[str, Any]:
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.rot_dims:
            out["rot"] = {"dims": self.rot_dims, "base": self.rot_base}
            if self.scaling is not None:
                out["rot"]["scaling"] = self.scaling.to_json()
        return out


@dataclass(frozen=True)
class NormedAttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    temp_coef: float
    temp_every: int

    @classmethod
    def read(cls, r: JsonReader) -> "NormedAttentionSizes":
        heads, kv = _heads(r)
        dim = r.integer("dim")
        t = _sub(r.raw, "q_temp", r.where, required=False)
        return cls(heads, kv, dim, r.integer("vdim", dim), r.number("scale"), t.number("coef", positive=False) if t else 0.0,
                   t.integer("every") if t else 1)

    def to_json(self) -> Dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
                "q_temp": {"coef": self.temp_coef, "every": self.temp_every}}


@dataclass(frozen=True)
class MatrixMemorySizes:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def read(cls, r: JsonReader) -> "MatrixMemorySizes":
        dim = r.integer("dim")
        return cls(r.integer("heads"), dim, r.integer("vdim", dim), r.number("gate_cap"))

    def to_json(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "gate_cap": self.gate_cap}


@dataclass(frozen=True)
class WeightedPairSizes:
    left: NormedAttentionSizes
    right: MatrixMemorySizes
    left_scale: float
    right_scale: float

    @classmethod
    def read(cls, r: JsonReader) -> "WeightedPairSizes":
        return cls(NormedAttentionSizes.read(_sub(r.raw, "left", r.where)), MatrixMemorySizes.read(_sub(r.raw, "right", r.where)),
                   r.number("left_scale", positive=False), r.number("right_scale", positive=False))

    def to_json(self) -> Dict[str, Any]:
        return {"left": self.left.to_json(), "right": self.right.to_json(), "left_scale": self.left_scale, "right_scale": self.right_scale}


@dataclass(frozen=True)
class LatentSinkAttentionSizes:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_base: float
    rot_dims: int

    @classmethod
    def read(cls, r: JsonReader) -> "LatentSinkAttentionSizes":
        rot = _sub(r.raw, "rot", r.where)
        rot_dim, dims = r.integer("rot_dim"), rot.integer("dims")
        if dims % 2 or dims > rot_dim:
            raise ConfigError(f"{r.where}: rot.dims {dims} must be even and at most rot_dim {rot_dim}")
        dim = r.integer("dim")
        return cls(r.integer("heads"), dim, rot_dim, r.integer("vdim", dim), r.integer("kv_rank"), r.integer("q_rank"), r.number("scale"),
                   rot.number("base"), dims)

    def to_json(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
                "q_rank": self.q_rank, "scale": self.scale, "rot": {"base": self.rot_base, "dims": self.rot_dims}}


_MIXERS = {"attention": RotaryAttentionSizes, "parallel": WeightedPairSizes, "latent_attention": LatentSinkAttentionSizes}


@dataclass(frozen=True)
class VarolixLayer:
    type: str
    mixer: Any  # one of the sizes above
    ff: Optional[int]  # the dense feed-forward's inner size; None: no feed-forward


@register_architecture("Varolix")
@dataclass(frozen=True)
class VarolixConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    layers: Tuple[VarolixLayer, ...]
    loop: Optional[LayerLoop]

    @classmethod
    def from_json(cls, raw: Mapping[str, Any]) -> "VarolixConfig":
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
            sizes = _MIXERS[kind].read(_sub(entry, "mixer", where))
            mlp = _sub(entry, "mlp", where, required=False)
            if mlp is not None and mlp.string("kind") != "dense":
                raise ConfigError(f"{where}.mlp: kind '{mlp.string('kind')}' is not supported (dense)")
            layers.append(VarolixLayer(kind, sizes, mlp.integer("ff") if mlp is not None else None))
        loop = _sub(raw, "loop", "config.json", required=False)
        if loop is not None:
            loop = LayerLoop(loop.integer("start", minimum=0), loop.integer("stop"), loop.integer("times"))
            if not loop.start < loop.stop <= len(layers):
                raise ConfigError(f"config.json.loop: layers {loop.start}..{loop.stop - 1} are not a range of the {len(layers)} layers")
        return cls(r.integer("vocab"), r.integer("width"), norm.number("eps"), tuple(layers), loop)

    def to_json(self) -> Dict[str, Any]:
        out = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
            "layers": [{"type": l.type, "mixer": l.mixer.to_json(), "mlp": {"kind": "dense", "ff": l.ff} if l.ff is not None else None}
                       for l in self.layers],
        }
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return out

    # ------------------------------------------------------------------ the model as data

    def _norm(self, name: str):
        return part("rmsnorm", tensor=name, size=self.width, eps=self.eps)

    def _mixer(self, layer: VarolixLayer, prefix: str):
        m = layer.mixer
        if layer.type == "attention":
            position = None
            if m.rot_dims:
                position = part("rope", head_dim=m.dim, rotary_dim=m.rot_dims, theta=m.rot_base, pairing="half",
                                scaling=m.scaling.to_json() if m.scaling is not None else None)
            return part("rotary_gated_attention", prefix=prefix, hidden_size=self.width, num_heads=m.heads, num_kv_heads=m.kv_heads,
                        key_dim=m.dim, value_dim=m.vdim, scale=m.scale, window=None, sink=False, head_gate=False, bias=True,
                        position=position)
        if layer.type == "latent_attention":
            return part("latent_attention", prefix=prefix, hidden_size=self.width, num_heads=m.heads, plain_dim=m.dim,
                        rotated_dim=m.rot_dim, value_dim=m.vdim, latent_dim=m.kv_rank, query_latent=m.q_rank, scale=m.scale,
                        eps=self.eps, window=None, gate="head", sink=True,
                        position=part("rope", head_dim=m.rot_dim, rotary_dim=m.rot_dims, theta=m.rot_base, pairing="half"))
        a, b = m.left, m.right
        left = part("chunked_attention", prefix=prefix + "left.", hidden_size=self.width, num_heads=a.heads, num_kv_heads=a.kv_heads,
                    key_dim=a.dim, value_dim=a.vdim, scale=a.scale, eps=self.eps, bias=True, value_bias=True, out_bias=True,
                    head_norm=True, norm_weight=True, temp_coef=a.temp_coef, temp_every=a.temp_every, max_positions=NO_POSITION_LIMIT)
        right = part("matrix_memory", prefix=prefix + "right.", hidden_size=self.width, num_heads=b.heads, key_dim=b.dim,
                     value_dim=b.vdim, gate_cap=b.gate_cap, eps=self.eps)
        return part("two_mixers", left=left, right=right, hidden_size=self.width, combine="weighted_sum", left_scale=m.left_scale,
                    right_scale=m.right_scale)

    def run_order(self) -> Tuple[RunSpec, ...]:
        """Every layer once, except that the looped range runs `times` times in a row; each run has its own cache or state."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(RunSpec(i) for i in range(n))
        lp = self.loop
        order = list(range(lp.start)) + list(range(lp.start, lp.stop)) * lp.times + list(range(lp.stop, n))
        return tuple(RunSpec(i) for i in order)

    def model_spec(self) -> ModelSpec:
        layers = []
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            ffn = None
            if layer.ff is not None:
                ffn = part("gated_mlp", prefix=p + "mlp.", hidden_size=self.width, intermediate_size=layer.ff, activation="gelu_tanh")
            layers.append(LayerSpec(block="prenorm", mixer=self._mixer(layer, p + "mix."), feed_forward=ffn,
                                    mixer_norm=self._norm(p + "norm1"), feed_forward_norm=self._norm(p + "norm2") if ffn else None,
                                    prefix=p))
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            embedding=part("embedding", tensor="embed", vocab_size=self.vocab, hidden_size=self.width),
            layers=tuple(layers), run_order=self.run_order(), final_norm=self._norm("final.norm"),
            head=part("lm_head", tensor="head", tied_to=None, vocab_size=self.vocab, hidden_size=self.width),
            max_positions=NO_POSITION_LIMIT,
        )
