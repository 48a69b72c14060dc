"""Typed configuration of the Mekazen decoder, read from ``config.json``.

A Mekazen model is a list of layers, each with sizes of its own. A layer is
norm -> attention -> norm -> residual sum, then (unless its ``mlp`` is null)
norm -> gated feed-forward -> norm -> residual sum. Its attention has no value
projection: the raw output of the key projection doubles as the values. q and
k are each normalised across all their heads at once, rotated in neighbouring
pairs over the first ``rot.dims`` values of a head (long wavelengths stretched
in three bands), masked so that a query only reaches back to the last absolute
multiple of ``mask.size``, and the heads' output is gated by a sigmoid. The
logits pass a tanh cap. The layers' and the model's norms are zero-centred in
the file (factor = 1 + w); the query and key norms hold the factor itself.

``config.json``::

    {"architecture": "Mekazen", "vocab": V, "width": W, "norm": {"eps": e},
     "logit_softcap": c,
     "layers": [{"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": s,
                           "mask": {"size": C},
                           "rot": {"base": b, "dims": R,
                                   "scaling": {"factor": f, "low": l, "high": h, "original": n}}},
                 "mlp": {"kind": "dense", "ff": F}}, ...]}

Tensors: ``embed`` [V, W]; per layer i ``l<i>.norm1``, ``l<i>.norm1b`` (and
``norm2``, ``norm2b`` with a feed-forward) [W]; ``l<i>.mix.q`` [H D, W],
``.k`` [G D, W], ``.g`` [H D, W], ``.o`` [W, H D], ``.q.norm`` [H D],
``.k.norm`` [G D]; ``l<i>.mlp.gate``, ``.up`` [F, W], ``.down`` [W, F];
``final.norm`` [W]; ``head`` [V, W].
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .qwen3 import ConfigError
from .spec import LayerRun, LayerSpec, ModelSpec, PartSpec

MAX_POSITIONS = 1 << 17   # the configuration names no limit; tables and graphs follow the engine's own


def _count(raw: Mapping[str, Any], key: str, where: str) -> int:
    value = raw.get(key)
    if isinstance(value, float) and value.is_integer():
        value = int(value)    # a writer that knows only one kind of number
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError("MissingDimension", f"{where}.{key} must be a positive integer, got {value!r}")
    return value


def _number(raw: Mapping[str, Any], key: str, where: str) -> float:
    value = raw.get(key)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(float(value)):
        raise ConfigError("Json", f"{where}.{key} must be a finite number, got {value!r}")
    return float(value)


def _object(value: Any, where: str) -> Mapping[str, Any]:
    if not isinstance(value, dict):
        raise ConfigError("Json", f"{where} must be an object, got {value!r}")
    return value


@dataclass(frozen=True)
class RotaryScaling:
    factor: float
    low: float
    high: float
    original: int

    def to_dict(self) -> Dict[str, Any]:
        return {"factor": self.factor, "high": self.high, "low": self.low, "original": self.original}


@dataclass(frozen=True)
class MekazenLayer:
    heads: int
    kv_heads: int
    dim: int
    scale: float
    chunk: int                       # 0: plain causal mask
    rotary_dims: int                 # 0: no rotation
    rotary_base: float
    rotary_scaling: Optional[RotaryScaling]
    ff: int                          # 0: no feed-forward

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "MekazenLayer":
        raw = _object(raw, where)
        kind = raw.get("type")
        if kind != "attention":
            raise ConfigError("UnsupportedLayerType", f"{where}.type {kind!r}; this design has 'attention' only")
        mixer = _object(raw.get("mixer"), f"{where}.mixer")
        at = f"{where}.mixer"
        heads, kv_heads, dim = (_count(mixer, key, at) for key in ("heads", "kv_heads", "dim"))
        if heads % kv_heads:
            raise ConfigError("InvalidGroupedQueryLayout", f"{at}: {heads} query heads over {kv_heads} key/value heads")
        if dim % 2:
            raise ConfigError("OddHeadDimension", f"{at}.dim {dim}")
        # the key projection's output serves as the values: one width for both
        if mixer.get("vdim", dim) != dim:
            raise ConfigError("InvalidValueWidth", f"{at}.vdim {mixer.get('vdim')!r} must equal dim {dim}")
        scale = _number(mixer, "scale", at)
        if scale <= 0.0:
            raise ConfigError("Json", f"{at}.scale must be positive, got {scale}")
        chunk = 0
        if mixer.get("mask") is not None:
            chunk = _count(_object(mixer["mask"], f"{at}.mask"), "size", f"{at}.mask")
        rotary_dims, base, scaling = 0, 0.0, None
        if mixer.get("rot") is not None:
            rot = _object(mixer["rot"], f"{at}.rot")
            rotary_dims = _count(rot, "dims", f"{at}.rot")
            if rotary_dims % 2 or rotary_dims > dim:
                raise ConfigError("InvalidRotaryWidth", f"{at}.rot.dims {rotary_dims} must be even and at most dim {dim}")
            base = _number(rot, "base", f"{at}.rot")
            if base <= 0.0:
                raise ConfigError("InvalidRopeTheta", f"{at}.rot.base {base}")
            if rot.get("scaling") is not None:
                s = _object(rot["scaling"], f"{at}.rot.scaling")
                scaling = RotaryScaling(factor=_number(s, "factor", f"{at}.rot.scaling"),
                                        low=_number(s, "low", f"{at}.rot.scaling"),
                                        high=_number(s, "high", f"{at}.rot.scaling"),
                                        original=_count(s, "original", f"{at}.rot.scaling"))
                if scaling.factor <= 0.0 or scaling.high <= scaling.low:
                    raise ConfigError("UnsupportedRopeScaling",
                                      f"{at}.rot.scaling needs factor > 0 and high > low, got {dict(s)}")
        ff = 0
        if raw.get("mlp") is not None:
            mlp = _object(raw["mlp"], f"{where}.mlp")
            if mlp.get("kind") != "dense":
                raise ConfigError("UnsupportedFeedForward", f"{where}.mlp.kind {mlp.get('kind')!r}; 'dense' only")
            ff = _count(mlp, "ff", f"{where}.mlp")
        return cls(heads=heads, kv_heads=kv_heads, dim=dim, scale=scale, chunk=chunk, rotary_dims=rotary_dims,
                   rotary_base=base, rotary_scaling=scaling, ff=ff)

    def to_dict(self) -> Dict[str, Any]:
        mixer: Dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads}
        if self.chunk:
            mixer["mask"] = {"size": self.chunk}
        if self.rotary_dims:
            rot: Dict[str, Any] = {"base": self.rotary_base, "dims": self.rotary_dims}
            if self.rotary_scaling is not None:
                rot["scaling"] = self.rotary_scaling.to_dict()
            mixer["rot"] = rot
        mixer["scale"] = self.scale
        mixer["vdim"] = self.dim
        return {"mixer": mixer, "mlp": {"ff": self.ff, "kind": "dense"} if self.ff else None, "type": "attention"}


@dataclass(frozen=True)
class MekazenConfig:
    """Sizes and constants of one Mekazen checkpoint."""

    vocab: int
    width: int
    norm_eps: float
    logit_softcap: float             # 0: the logits are not capped
    layers: Tuple[MekazenLayer, ...]
    eos_token_ids: tuple = ()

    ARCHITECTURE = "Mekazen"
    MODEL_TYPE = "mekazen"

    @classmethod
    def parse(cls, text: str) -> "MekazenConfig":
        try:
            raw = json.loads(text)
        except json.JSONDecodeError as error:
            raise ConfigError("Json", str(error)) from None
        return cls.from_dict(_object(raw, "config.json"))

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "MekazenConfig":
        if raw.get("architecture") != cls.ARCHITECTURE:
            raise ConfigError("UnsupportedModelType", f"architecture {raw.get('architecture')!r}")
        vocab, width = _count(raw, "vocab", "config"), _count(raw, "width", "config")
        eps = _number(_object(raw.get("norm"), "norm"), "eps", "norm")   # kernels take it rounded to 32 bits
        if eps <= 0.0:
            raise ConfigError("InvalidRmsNormEpsilon", str(eps))
        cap = 0.0
        if raw.get("logit_softcap"):     # absent, null or 0: no cap
            cap = _number(raw, "logit_softcap", "config")
            if cap <= 0.0:
                raise ConfigError("Json", f"logit_softcap must be positive, got {cap}")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("MissingDimension", "layers must be a list of at least one layer")
        return cls(vocab=vocab, width=width, norm_eps=eps, logit_softcap=cap,
                   layers=tuple(MekazenLayer.from_dict(layer, f"layers[{i}]") for i, layer in enumerate(layers)))

    # ------------------------------------------------------------ derived facts
    @property
    def vocab_size(self) -> int:      # the names every family answers to
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    def kv_bytes_per_token(self, bytes_per_value: int) -> int:
        return sum(2 * layer.kv_heads * layer.dim * bytes_per_value for layer in self.layers)

    def parameter_count(self) -> int:
        return sum(math.prod(shape) for shape in self.tensor_shapes().values())

    def to_dict(self) -> Dict[str, Any]:
        """The ``config.json`` this configuration is read back from."""
        out: Dict[str, Any] = {"architecture": self.ARCHITECTURE,
                               "layers": [layer.to_dict() for layer in self.layers]}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        out.update(norm={"eps": self.norm_eps}, vocab=self.vocab, width=self.width)
        return out

    # ------------------------------------------------------------- model spec
    def to_model_spec(self) -> ModelSpec:
        w, eps = self.width, self.norm_eps
        stored_around_zero = lambda name, size=w: PartSpec("rmsnorm", {
            "size": size, "eps": eps, "weight": name, "one_plus": True})
        layers = []
        for index, layer in enumerate(self.layers):
            base = f"l{index}"
            q_size, kv_size = layer.heads * layer.dim, layer.kv_heads * layer.dim
            position = None
            if layer.rotary_dims:
                position = PartSpec("rope_interleaved", {
                    "theta": layer.rotary_base, "rotary_dim": layer.rotary_dims, "head_dim": layer.dim,
                    "scaling": layer.rotary_scaling.to_dict() if layer.rotary_scaling else None})
            mixer = PartSpec("gqa_attention", {
                "hidden_size": w, "num_heads": layer.heads, "num_kv_heads": layer.kv_heads,
                "head_dim": layer.dim, "scale": layer.scale, "window": None, "chunk": layer.chunk or None,
                "q_proj": f"{base}.mix.q", "k_proj": f"{base}.mix.k", "v_proj": None,
                "gate_proj": f"{base}.mix.g", "o_proj": f"{base}.mix.o",
                "qk_norm_scope": "projection",
                "q_norm": PartSpec("rmsnorm", {"size": q_size, "eps": eps, "weight": f"{base}.mix.q.norm"}),
                "k_norm": PartSpec("rmsnorm", {"size": kv_size, "eps": eps, "weight": f"{base}.mix.k.norm"}),
                "position": position})
            feed_forward = None
            if layer.ff:
                feed_forward = PartSpec("swiglu", {
                    "hidden_size": w, "intermediate_size": layer.ff, "gate_proj": f"{base}.mlp.gate",
                    "up_proj": f"{base}.mlp.up", "down_proj": f"{base}.mlp.down"})
            layers.append(LayerSpec(
                name=base, block=PartSpec("sandwich_residual", {}), mixer=mixer, feed_forward=feed_forward,
                mixer_norm=stored_around_zero(f"{base}.norm1"),
                mixer_post_norm=stored_around_zero(f"{base}.norm1b"),
                feed_forward_norm=stored_around_zero(f"{base}.norm2") if layer.ff else None,
                feed_forward_post_norm=stored_around_zero(f"{base}.norm2b") if layer.ff else None))
        spec = ModelSpec(
            architecture=self.ARCHITECTURE, hidden_size=w, vocab_size=self.vocab, max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": w, "weight": "embed"}),
            layers=tuple(layers), order=tuple(LayerRun(layer=i) for i in range(len(layers))),
            final_norm=stored_around_zero("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": w, "weight": "head",
                                          "softcap": self.logit_softcap or None}))
        spec.validate()
        return spec

    # ------------------------------------------------ tensors of a checkpoint
    def tensor_shapes(self) -> Dict[str, tuple]:
        w = self.width
        shapes: Dict[str, tuple] = {"embed": (self.vocab, w)}
        for index, layer in enumerate(self.layers):
            base = f"l{index}"
            q_size, kv_size = layer.heads * layer.dim, layer.kv_heads * layer.dim
            names = ("norm1", "norm2", "norm1b", "norm2b") if layer.ff else ("norm1", "norm1b")
            shapes.update({f"{base}.{name}": (w,) for name in names})
            shapes.update({f"{base}.mix.q": (q_size, w), f"{base}.mix.k": (kv_size, w),
                           f"{base}.mix.q.norm": (q_size,), f"{base}.mix.k.norm": (kv_size,),
                           f"{base}.mix.g": (q_size, w), f"{base}.mix.o": (w, q_size)})
            if layer.ff:
                shapes.update({f"{base}.mlp.gate": (layer.ff, w), f"{base}.mlp.up": (layer.ff, w),
                               f"{base}.mlp.down": (w, layer.ff)})
        shapes["final.norm"] = (w,)
        shapes["head"] = (self.vocab, w)
        return shapes

    def ignored_tensors(self) -> tuple:
        """The second pair of norms of a layer without a feed-forward, should a
        checkpoint hold them all the same: nothing reads them."""
        return tuple(f"l{index}.{name}" for index, layer in enumerate(self.layers) if not layer.ff
                     for name in ("norm2", "norm2b"))

    def norm_tensor(self, name: str):
        """False for a matrix; for a norm weight how it is stored: "one" (the
        factor itself) or "zero" (the factor is 1 + w)."""
        if name.endswith(".q.norm") or name.endswith(".k.norm"):
            return "one"
        last = name.rsplit(".", 1)[-1]
        return "zero" if last in ("norm1", "norm2", "norm1b", "norm2b", "norm") else False
