"""Typed configuration of the Zitezen decoder, read from ``config.json``.

A Zitezen model keeps ``streams`` copies of the residual stream
(hyper-connections): every sublayer reads a weighted sum of them, runs on its
Dynamic Tanh norm (tanh(alpha u) w + b), and its result, times a per-channel
layer scale, is written back to all of them through a small mixing matrix. A
layer has one of three mixers and, unless its ``mlp`` is null, a feed-forward
down(relu(up(h))^2):

* ``mlstm``: a matrix-memory recurrence per head with capped, exponential
  input and forget gates, a per-head RMS norm and a sigmoid output gate;
* ``latent_attention``: causal softmax attention whose keys and values are
  up-projected from one cached latent per position, with a small rotated key
  part shared by all heads (rotation of neighbouring pairs);
* ``parallel``: grouped-query attention (per-head q/k RMS norm, rotation of
  the halves of the first ``rot.dims`` values, capped scores, one sigmoid gate
  per head) beside an ``mlstm``, their results added with fixed weights.

``loop`` {start, stop, times} runs layers start .. stop-1 that many times in a
row with the same weights; every pass has cache entries of its own.

``config.json``::

    {"architecture": "Zitezen", "vocab": V, "width": W, "streams": S, "norm": {"eps": e},
     "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "mlstm", "mixer": {"heads": H, "dim": D, "vdim": Dv, "gate_cap": c}, "mlp": null},
                {"type": "latent_attention",
                 "mixer": {"heads": H, "dim": D, "rot_dim": R, "vdim": Dv, "kv_rank": r, "q_rank": rq,
                           "scale": s, "rot": {"base": b, "dims": R}},
                 "mlp": {"kind": "dense", "ff": F}},
                {"type": "parallel",
                 "mixer": {"left": {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": s, "softcap": c,
                                    "rot": {"base": b, "dims": Rd}},
                           "right": {"heads": H, "dim": D, "vdim": Dv, "gate_cap": c},
                           "left_scale": x, "right_scale": y},
                 "mlp": {"kind": "dense", "ff": F}}]}

Tensors (linear weights ``[out, in]``): ``embed`` [V, W], ``head`` [V, W],
``final.norm`` [W] with ``.b`` [W] and ``.alpha`` []; per layer i
``l<i>.norm1`` (and ``norm2`` with a feed-forward) likewise, ``l<i>.ls1``,
``ls2`` [W], ``l<i>.hc1.in``, ``.out`` [S], ``.mix`` [S, S] (and ``hc2``),
``l<i>.mlp.up`` [F, W], ``.down`` [W, F]; under ``l<i>.mix`` an mlstm has
``q``, ``k`` [H D, W], ``v``, ``g`` [H Dv, W], ``o`` [W, H Dv], ``norm``
[H Dv], ``i``, ``f`` [H, W], ``i.b``, ``f.b`` [H]; a latent attention ``dq``
[rq, W], ``dq.norm`` [rq], ``uq`` [H (D + R), rq], ``dkv`` [r + R, W],
``dkv.norm`` [r], ``uk`` [H D, r], ``uv`` [H Dv, r], ``o`` [W, H Dv]; a
parallel mixer ``left.q`` [H D, W], ``left.k`` [G D, W], ``left.v`` [G Dv, W],
``left.q.norm``, ``left.k.norm`` [D], ``left.g`` [H, W], ``left.o`` [W, H Dv]
and an mlstm's tensors under ``right``.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .mekazen import MAX_POSITIONS, _count, _number, _object
from .qwen3 import ConfigError
from .spec import LayerRun, LayerSpec, ModelSpec, PartSpec


def _rotation(raw: Mapping[str, Any], where: str, limit: int) -> Tuple[int, float]:
    """(dims, base) of an optional ``rot`` object; (0, 0.0) without one."""
    if raw.get("rot") is None:
        return 0, 0.0
    rot = _object(raw["rot"], f"{where}.rot")
    dims = _count(rot, "dims", f"{where}.rot")
    if dims % 2 or dims > limit:
        raise ConfigError("InvalidRotaryWidth", f"{where}.rot.dims {dims} must be even and at most {limit}")
    base = _number(rot, "base", f"{where}.rot")
    if base <= 0.0:
        raise ConfigError("InvalidRopeTheta", f"{where}.rot.base {base}")
    return dims, base


def _positive(raw: Mapping[str, Any], key: str, where: str) -> float:
    value = _number(raw, key, where)
    if value <= 0.0:
        raise ConfigError("Json", f"{where}.{key} must be positive, got {value}")
    return value


@dataclass(frozen=True)
class MatrixMemoryMixer:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "MatrixMemoryMixer":
        raw = _object(raw, where)
        return cls(heads=_count(raw, "heads", where), dim=_count(raw, "dim", where), vdim=_count(raw, "vdim", where),
                   gate_cap=_positive(raw, "gate_cap", where))

    def to_dict(self) -> Dict[str, Any]:
        return {"dim": self.dim, "gate_cap": self.gate_cap, "heads": self.heads, "vdim": self.vdim}

    def shapes(self, base: str, w: int) -> Dict[str, tuple]:
        k, v = self.heads * self.dim, self.heads * self.vdim
        return {f"{base}.q": (k, w), f"{base}.k": (k, w), f"{base}.v": (v, w), f"{base}.g": (v, w),
                f"{base}.o": (w, v), f"{base}.norm": (v,), f"{base}.i": (self.heads, w), f"{base}.i.b": (self.heads,),
                f"{base}.f": (self.heads, w), f"{base}.f.b": (self.heads,)}

    def part(self, base: str, w: int, eps: float) -> PartSpec:
        return PartSpec("mlstm", {
            "hidden_size": w, "num_heads": self.heads, "head_dim": self.dim, "value_dim": self.vdim,
            "gate_cap": self.gate_cap, "eps": eps, "q_proj": f"{base}.q", "k_proj": f"{base}.k",
            "v_proj": f"{base}.v", "gate_proj": f"{base}.g", "o_proj": f"{base}.o", "norm": f"{base}.norm",
            "input_gate_proj": f"{base}.i", "input_gate_bias": f"{base}.i.b",
            "forget_gate_proj": f"{base}.f", "forget_gate_bias": f"{base}.f.b"})


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rotary_dims: int
    rotary_base: float

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "LatentMixer":
        raw = _object(raw, where)
        rot_dim = _count(raw, "rot_dim", where)
        dims, base = _rotation(raw, where, rot_dim)
        return cls(heads=_count(raw, "heads", where), dim=_count(raw, "dim", where), rot_dim=rot_dim,
                   vdim=_count(raw, "vdim", where), kv_rank=_count(raw, "kv_rank", where),
                   q_rank=_count(raw, "q_rank", where), scale=_positive(raw, "scale", where),
                   rotary_dims=dims, rotary_base=base)

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "q_rank": self.q_rank}
        if self.rotary_dims:
            out["rot"] = {"base": self.rotary_base, "dims": self.rotary_dims}
        out.update(rot_dim=self.rot_dim, scale=self.scale, vdim=self.vdim)
        return out

    def shapes(self, base: str, w: int) -> Dict[str, tuple]:
        h = self.heads
        return {f"{base}.dq": (self.q_rank, w), f"{base}.dq.norm": (self.q_rank,),
                f"{base}.uq": (h * (self.dim + self.rot_dim), self.q_rank),
                f"{base}.dkv": (self.kv_rank + self.rot_dim, w), f"{base}.dkv.norm": (self.kv_rank,),
                f"{base}.uk": (h * self.dim, self.kv_rank), f"{base}.uv": (h * self.vdim, self.kv_rank),
                f"{base}.o": (w, h * self.vdim)}

    def part(self, base: str, w: int, eps: float, cache_mode: str = "auto") -> PartSpec:
        position = None
        if self.rotary_dims:
            position = PartSpec("rope_interleaved", {"theta": self.rotary_base, "rotary_dim": self.rotary_dims,
                                                     "head_dim": self.rot_dim, "scaling": None})
        return PartSpec("latent_attention", {
            "cache_mode": cache_mode,
            "hidden_size": w, "num_heads": self.heads, "head_dim": self.dim, "rotary_head_dim": self.rot_dim,
            "value_dim": self.vdim, "kv_rank": self.kv_rank, "q_rank": self.q_rank, "scale": self.scale, "eps": eps,
            "q_down_proj": f"{base}.dq", "q_up_proj": f"{base}.uq", "kv_down_proj": f"{base}.dkv",
            "k_up_proj": f"{base}.uk", "v_up_proj": f"{base}.uv", "o_proj": f"{base}.o",
            "q_norm": PartSpec("rmsnorm", {"size": self.q_rank, "eps": eps, "weight": f"{base}.dq.norm"}),
            "kv_norm": PartSpec("rmsnorm", {"size": self.kv_rank, "eps": eps, "weight": f"{base}.dkv.norm"}),
            "position": position})


@dataclass(frozen=True)
class GroupedMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float          # 0: the scores are not capped
    rotary_dims: int
    rotary_base: float

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "GroupedMixer":
        raw = _object(raw, where)
        heads, dim = _count(raw, "heads", where), _count(raw, "dim", where)
        kv_heads = _count(raw, "kv_heads", where) if raw.get("kv_heads") is not None else heads
        if heads % kv_heads:
            raise ConfigError("InvalidGroupedQueryLayout", f"{where}: {heads} query heads over {kv_heads} key/value heads")
        dims, base = _rotation(raw, where, dim)
        cap = _positive(raw, "softcap", where) if raw.get("softcap") else 0.0
        return cls(heads=heads, kv_heads=kv_heads, dim=dim, vdim=_count(raw, "vdim", where),
                   scale=_positive(raw, "scale", where), softcap=cap, rotary_dims=dims, rotary_base=base)

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads}
        if self.rotary_dims:
            out["rot"] = {"base": self.rotary_base, "dims": self.rotary_dims}
        out["scale"] = self.scale
        if self.softcap:
            out["softcap"] = self.softcap
        out["vdim"] = self.vdim
        return out

    def shapes(self, base: str, w: int) -> Dict[str, tuple]:
        return {f"{base}.q": (self.heads * self.dim, w), f"{base}.k": (self.kv_heads * self.dim, w),
                f"{base}.v": (self.kv_heads * self.vdim, w), f"{base}.q.norm": (self.dim,),
                f"{base}.k.norm": (self.dim,), f"{base}.g": (self.heads, w), f"{base}.o": (w, self.heads * self.vdim)}

    def part(self, base: str, w: int, eps: float) -> PartSpec:
        position = None
        if self.rotary_dims:
            position = PartSpec("rope_half", {"theta": self.rotary_base, "rotary_dim": self.rotary_dims,
                                              "head_dim": self.dim, "scaling": None})
        return PartSpec("gqa_attention", {
            "hidden_size": w, "num_heads": self.heads, "num_kv_heads": self.kv_heads, "head_dim": self.dim,
            "value_dim": self.vdim, "scale": self.scale, "softcap": self.softcap or None, "window": None,
            "chunk": None, "q_proj": f"{base}.q", "k_proj": f"{base}.k", "v_proj": f"{base}.v",
            "gate_proj": f"{base}.g", "gate_scope": "head", "o_proj": f"{base}.o", "qk_norm_scope": "head",
            "q_norm": PartSpec("rmsnorm", {"size": self.dim, "eps": eps, "weight": f"{base}.q.norm"}),
            "k_norm": PartSpec("rmsnorm", {"size": self.dim, "eps": eps, "weight": f"{base}.k.norm"}),
            "position": position})


@dataclass(frozen=True)
class ParallelMixer:
    left: GroupedMixer
    right: MatrixMemoryMixer
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "ParallelMixer":
        raw = _object(raw, where)
        return cls(left=GroupedMixer.from_dict(raw.get("left"), f"{where}.left"),
                   right=MatrixMemoryMixer.from_dict(raw.get("right"), f"{where}.right"),
                   left_scale=_number(raw, "left_scale", where), right_scale=_number(raw, "right_scale", where))

    def to_dict(self) -> Dict[str, Any]:
        return {"left": self.left.to_dict(), "left_scale": self.left_scale, "right": self.right.to_dict(),
                "right_scale": self.right_scale}

    def shapes(self, base: str, w: int) -> Dict[str, tuple]:
        return {**self.left.shapes(f"{base}.left", w), **self.right.shapes(f"{base}.right", w)}

    def part(self, base: str, w: int, eps: float) -> PartSpec:
        return PartSpec("parallel_mixers", {
            "left": self.left.part(f"{base}.left", w, eps), "right": self.right.part(f"{base}.right", w, eps),
            "left_scale": self.left_scale, "right_scale": self.right_scale})


_MIXERS = {"mlstm": MatrixMemoryMixer, "latent_attention": LatentMixer, "parallel": ParallelMixer}


@dataclass(frozen=True)
class ZitezenLayer:
    kind: str                # "mlstm", "latent_attention" or "parallel"
    mixer: object
    ff: int                  # 0: no feed-forward

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "ZitezenLayer":
        raw = _object(raw, where)
        kind = raw.get("type")
        if kind not in _MIXERS:
            raise ConfigError("UnsupportedLayerType", f"{where}.type {kind!r}; this design has {sorted(_MIXERS)}")
        ff = 0
        if raw.get("mlp") is not None:
            mlp = _object(raw["mlp"], f"{where}.mlp")
            if mlp.get("kind") != "dense":
                raise ConfigError("UnsupportedFeedForward", f"{where}.mlp.kind {mlp.get('kind')!r}; 'dense' only")
            ff = _count(mlp, "ff", f"{where}.mlp")
        return cls(kind=kind, mixer=_MIXERS[kind].from_dict(raw.get("mixer"), f"{where}.mixer"), ff=ff)

    def to_dict(self) -> Dict[str, Any]:
        return {"mixer": self.mixer.to_dict(), "mlp": {"ff": self.ff, "kind": "dense"} if self.ff else None,
                "type": self.kind}


@dataclass(frozen=True)
class ZitezenConfig:
    """Sizes and constants of one Zitezen checkpoint."""

    vocab: int
    width: int
    streams: int
    norm_eps: float
    layers: Tuple[ZitezenLayer, ...]
    loop: Optional[Tuple[int, int, int]] = None      # (start, stop, times)
    eos_token_ids: tuple = ()

    ARCHITECTURE = "Zitezen"
    MODEL_TYPE = "zitezen"
    MAX_STREAMS = 8

    @classmethod
    def parse(cls, text: str) -> "ZitezenConfig":
        try:
            raw = json.loads(text)
        except json.JSONDecodeError as error:
            raise ConfigError("Json", str(error)) from None
        return cls.from_dict(_object(raw, "config.json"))

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "ZitezenConfig":
        if raw.get("architecture") != cls.ARCHITECTURE:
            raise ConfigError("UnsupportedModelType", f"architecture {raw.get('architecture')!r}")
        vocab, width = _count(raw, "vocab", "config"), _count(raw, "width", "config")
        streams = _count(raw, "streams", "config") if raw.get("streams") is not None else 1
        if streams > cls.MAX_STREAMS:
            raise ConfigError("Json", f"streams {streams}: up to {cls.MAX_STREAMS} residual streams are taken")
        eps = _number(_object(raw.get("norm"), "norm"), "eps", "norm")
        if eps <= 0.0:
            raise ConfigError("InvalidRmsNormEpsilon", str(eps))
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("MissingDimension", "layers must be a list of at least one layer")
        loop = None
        if raw.get("loop") is not None:
            spec = _object(raw["loop"], "loop")
            times = _count(spec, "times", "loop")
            start, stop = spec.get("start"), spec.get("stop")
            for key, value in (("start", start), ("stop", stop)):
                if isinstance(value, bool) or not isinstance(value, int):
                    raise ConfigError("Json", f"loop.{key} must be an integer, got {value!r}")
            if not 0 <= start <= stop <= len(layers):
                raise ConfigError("Json", f"loop {start}..{stop} does not lie within the {len(layers)} layers")
            loop = (start, stop, times)
        return cls(vocab=vocab, width=width, streams=streams, norm_eps=eps, loop=loop,
                   layers=tuple(ZitezenLayer.from_dict(layer, f"layers[{i}]") for i, layer in enumerate(layers)))

    # ------------------------------------------------------------ derived facts
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    def layer_order(self) -> Tuple[int, ...]:
        """Layer indices in the order they run, a looped stretch repeated."""
        count = len(self.layers)
        if self.loop is None:
            return tuple(range(count))
        start, stop, times = self.loop
        return tuple(range(start)) + tuple(range(start, stop)) * times + tuple(range(stop, count))

    def parameter_count(self) -> int:
        return sum(math.prod(shape) for shape in self.tensor_shapes().values())

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": self.ARCHITECTURE, "layers": [layer.to_dict() for layer in self.layers]}
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        out.update(norm={"eps": self.norm_eps}, streams=self.streams, vocab=self.vocab, width=self.width)
        return out

    # ------------------------------------------------------------- model spec
    def to_model_spec(self, latent_cache: str = "auto") -> ModelSpec:
        """``latent_cache``: what the latent attention keeps per position: "latent"
        (the shared latent row), "heads" (every head's key and value rows) or
        "auto" (the latter where the tensor-core kernels take the head size)."""
        w, eps, s = self.width, self.norm_eps, self.streams
        norm = lambda name: PartSpec("dynamic_tanh", {"size": w, "weight": name, "bias": f"{name}.b",
                                                      "alpha": f"{name}.alpha"})
        connection = lambda base, q: {"in": f"{base}.hc{q}.in", "out": f"{base}.hc{q}.out",
                                      "mix": f"{base}.hc{q}.mix", "scale": f"{base}.ls{q}"}
        layers = []
        for index, layer in enumerate(self.layers):
            base = f"l{index}"
            feed_forward = None
            block = {"streams": s, "hidden_size": w, "mixer": connection(base, 1)}
            if layer.ff:
                feed_forward = PartSpec("dense_ff", {
                    "hidden_size": w, "intermediate_size": layer.ff, "activation": "relu_squared",
                    "up_proj": f"{base}.mlp.up", "down_proj": f"{base}.mlp.down"})
                block["feed_forward"] = connection(base, 2)
            layers.append(LayerSpec(
                name=base, block=PartSpec("hyper_connections", block),
                mixer=layer.mixer.part(f"{base}.mix", w, eps, latent_cache) if layer.kind == "latent_attention"
                else layer.mixer.part(f"{base}.mix", w, eps),
                feed_forward=feed_forward, mixer_norm=norm(f"{base}.norm1"),
                feed_forward_norm=norm(f"{base}.norm2") if layer.ff else None))
        # every run of a layer, a repeated one too, keeps what it caches in an entry of its own
        order = tuple(LayerRun(layer=layer, cache=run) for run, layer in enumerate(self.layer_order()))
        spec = ModelSpec(
            architecture=self.ARCHITECTURE, hidden_size=w, vocab_size=self.vocab, max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": w, "weight": "embed"}),
            layers=tuple(layers), order=order, final_norm=norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": w, "weight": "head",
                                          "softcap": None}),
            streams=s)
        spec.validate()
        return spec

    # ------------------------------------------------ tensors of a checkpoint
    def tensor_shapes(self) -> Dict[str, tuple]:
        w, s = self.width, self.streams
        shapes: Dict[str, tuple] = {"embed": (self.vocab, w)}
        norm = lambda name: {name: (w,), f"{name}.b": (w,), f"{name}.alpha": ()}
        for index, layer in enumerate(self.layers):
            base = f"l{index}"
            shapes.update(norm(f"{base}.norm1"))
            if layer.ff:
                shapes.update(norm(f"{base}.norm2"))
            shapes.update(layer.mixer.shapes(f"{base}.mix", w))
            if layer.ff:
                shapes.update({f"{base}.mlp.up": (layer.ff, w), f"{base}.mlp.down": (w, layer.ff)})
            for q in (1, 2) if layer.ff else (1,):
                shapes[f"{base}.ls{q}"] = (w,)
            for q in (1, 2) if layer.ff else (1,):
                shapes.update({f"{base}.hc{q}.in": (s,), f"{base}.hc{q}.out": (s,), f"{base}.hc{q}.mix": (s, s)})
        shapes.update(norm("final.norm"))
        shapes["head"] = (self.vocab, w)
        return shapes

    def ignored_tensors(self) -> tuple:
        """The second sublayer's tensors of a layer without a feed-forward,
        should a checkpoint hold them all the same: nothing reads them."""
        names = []
        for index, layer in enumerate(self.layers):
            if not layer.ff:
                names += [f"l{index}.{name}" for name in ("norm2", "norm2.b", "norm2.alpha", "ls2", "hc2.in",
                                                          "hc2.out", "hc2.mix")]
        return tuple(names)

    def norm_tensor(self, name: str):
        """How a tensor of random weights is drawn: False for a matrix
        (N(0, 0.02)); "one" for a factor near 1; "zero" for an offset near 0;
        "identity" for a small square matrix near the identity."""
        last = name.rsplit(".", 1)[-1]
        if last == "mix" and ".hc" in name:
            return "identity"
        if last == "b":
            return "zero"
        if last in ("norm1", "norm2", "norm", "alpha", "ls1", "ls2", "in", "out"):
            return "one"
        return False
