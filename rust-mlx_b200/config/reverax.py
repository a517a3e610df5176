"""Configuration of the Reverax decoder.

config.json of this family is nested:

    architecture      "Reverax"
    vocab, width
    norm.eps, norm.groups   every norm of the stream: the row in `groups` equal consecutive parts, each over its own root mean
                            square (groups absent: 1); eps is also the eps of the norms inside the mixers
    logit_scale       what the logits are multiplied with (absent: 1)
    layers[]          one entry a layer, in order:
        type          "attention" or "parallel"
        weights_of    optional: the index of an earlier layer whose tensors this layer uses (mixer, feed-forward, norms, scales),
                      with caches and states of its own; the rest of the entry equals that layer's
        mixer         attention: heads, kv_heads, dim (query/key numbers a head), vdim, scale, rot: base, dims
                      parallel:  left (heads, kv_heads, dim, vdim, scale, softcap (optional), mask.size (optional: a window),
                                 rot: base, dims), right (heads, dim; rank optional), left_scale, right_scale
        mlp           null, or kind "dense": ff;  or kind "moe": expert.ff, router.experts, router.top

One size is not in config.json: the inner size of the decay's two small products of a "parallel" layer's right mixer
(``right.rank``).  A checkpoint's folder gives it through the shape of ``l<i>.mix.right.w1`` (``sizes_from_tensors``); a
configuration that is written out (``to_dict``) names it, so that a model made from a configuration alone has it too.

Every other size and constant is read from config.json; every problem of a file is reported in one ``ConfigError``.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Optional

from .base import ConfigError, ModelConfig
from .resolorn import _float, _int

MIXERS = ("attention", "parallel")


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int

    def to_dict(self) -> dict:
        return {"base": self.base, "dims": self.dims}


@dataclass(frozen=True)
class TalkingAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Rotation

    def to_dict(self) -> dict:
        return {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "rot": self.rot.to_dict(), "scale": self.scale,
                "vdim": self.vdim}


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Rotation
    softcap: float = 0.0        # 0: none
    window: int = 0             # 0: every earlier position is read

    def to_dict(self) -> dict:
        out = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "rot": self.rot.to_dict(), "scale": self.scale,
               "vdim": self.vdim}
        if self.window:
            out["mask"] = {"size": self.window}
        if self.softcap:
            out["softcap"] = self.softcap
        return out


@dataclass(frozen=True)
class TimeMixConfig:
    heads: int
    dim: int
    rank: int = 0               # 0: not known yet (a checkpoint's tensor gives it)

    def to_dict(self) -> dict:
        out = {"dim": self.dim, "heads": self.heads}
        if self.rank:
            out["rank"] = self.rank
        return out


@dataclass(frozen=True)
class SideBySideConfig:
    left: WindowAttentionConfig
    right: TimeMixConfig
    left_scale: float
    right_scale: float

    def to_dict(self) -> dict:
        return {"left": self.left.to_dict(), "left_scale": self.left_scale, "right": self.right.to_dict(), "right_scale": self.right_scale}


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                   # "dense" or "moe"
    ff: int
    experts: int = 0
    top: int = 0

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense"}
        return {"expert": {"ff": self.ff}, "kind": "moe", "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class ReveraxLayer:
    type: str
    mixer: object
    mlp: Optional[FeedForwardConfig]
    weights_of: Optional[int] = None

    def to_dict(self) -> dict:
        out = {"mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp is not None else None, "type": self.type}
        if self.weights_of is not None:
            out["weights_of"] = self.weights_of
        return out


def _rotation(p, where, m) -> Rotation:
    rot = m.get("rot")
    if not isinstance(rot, dict):
        p.append(f"{where}: missing 'rot' (an object with 'base' and 'dims')")
        return Rotation(10000.0, 0)
    return Rotation(_float(p, f"{where}.rot", rot, "base"), _int(p, f"{where}.rot", rot, "dims", minimum=0))


def _attention(p, w, m, windowed: bool):
    common = dict(heads=_int(p, w, m, "heads"), kv_heads=_int(p, w, m, "kv_heads"), dim=_int(p, w, m, "dim"),
                  vdim=_int(p, w, m, "vdim"), scale=_float(p, w, m, "scale"), rot=_rotation(p, w, m))
    if not windowed:
        return TalkingAttentionConfig(**common)
    mask = m.get("mask")
    return WindowAttentionConfig(softcap=_float(p, w, m, "softcap", required=False, default=0.0),
                                 window=_int(p, f"{w}.mask", mask, "size") if isinstance(mask, dict) else 0, **common)


@dataclass
class ReveraxConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    eps: float = 0.0
    norm_groups: int = 1
    logit_scale: float = 1.0
    layers: tuple = ()
    eos_token_id: tuple = ()

    @classmethod
    def from_dict(cls, raw: dict) -> "ReveraxConfig":
        if not isinstance(raw, dict):
            raise ConfigError("config.json must hold a JSON object")
        p = []
        name = raw.get("architecture") or (raw.get("architectures") or [""])[0]
        vocab = _int(p, "config", raw, "vocab")
        width = _int(p, "config", raw, "width")
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            p.append("config: missing 'norm' (an object with 'eps')")
            norm = {}
        eps = _float(p, "norm", norm, "eps", required=isinstance(raw.get("norm"), dict))
        groups = _int(p, "norm", norm, "groups", required=False, default=1)
        logit_scale = _float(p, "config", raw, "logit_scale", required=False, default=1.0)
        entries = raw.get("layers")
        layers = []
        if not isinstance(entries, list) or not entries:
            p.append("config: 'layers' must be a list with at least one layer")
            entries = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]"
            if not isinstance(entry, dict):
                p.append(f"{where}: must be an object")
                continue
            kind = entry.get("type")
            if kind not in MIXERS:
                p.append(f"{where}: unknown mixer type {kind!r} (known: {', '.join(MIXERS)})")
                continue
            m = entry.get("mixer")
            if not isinstance(m, dict):
                p.append(f"{where}: missing 'mixer'")
                continue
            w = f"{where}.mixer"
            if kind == "attention":
                mixer = _attention(p, w, m, windowed=False)
            else:
                left, right = m.get("left"), m.get("right")
                if not isinstance(left, dict) or not isinstance(right, dict):
                    p.append(f"{w}: a parallel mixer has 'left' and 'right'")
                    continue
                mixer = SideBySideConfig(
                    left=_attention(p, f"{w}.left", left, windowed=True),
                    right=TimeMixConfig(heads=_int(p, f"{w}.right", right, "heads"), dim=_int(p, f"{w}.right", right, "dim"),
                                        rank=_int(p, f"{w}.right", right, "rank", required=False, default=0)),
                    left_scale=_float(p, w, m, "left_scale", required=False, default=1.0),
                    right_scale=_float(p, w, m, "right_scale", required=False, default=1.0))
            f = entry.get("mlp")
            mlp = None
            if f is not None:
                if not isinstance(f, dict) or f.get("kind") not in ("dense", "moe"):
                    p.append(f"{where}.mlp: 'kind' must be 'dense' or 'moe' (or the layer's 'mlp' null)")
                elif f["kind"] == "dense":
                    mlp = FeedForwardConfig("dense", _int(p, f"{where}.mlp", f, "ff"))
                else:
                    router = f.get("router") if isinstance(f.get("router"), dict) else {}
                    mlp = FeedForwardConfig("moe", _int(p, f"{where}.mlp.expert", f.get("expert"), "ff"),
                                            experts=_int(p, f"{where}.mlp.router", router, "experts"),
                                            top=_int(p, f"{where}.mlp.router", router, "top"))
            shared = entry.get("weights_of")
            if shared is not None and (isinstance(shared, bool) or not isinstance(shared, int)):
                p.append(f"{where}: 'weights_of' must be a layer's index")
                shared = None
            layers.append(ReveraxLayer(kind, mixer, mlp, shared))
        if p:
            raise ConfigError("invalid configuration: " + "; ".join(p))
        eos = raw.get("eos_token_id")
        eos = () if eos is None else (tuple(eos) if isinstance(eos, (list, tuple)) else (eos,))
        cfg = cls(model_type="reverax", architectures=(name or "Reverax",), vocab=vocab, width=width, eps=eps, norm_groups=groups,
                  logit_scale=logit_scale, layers=tuple(layers), eos_token_id=eos)
        cfg._raw = dict(raw)
        p = cfg.validate()
        if p:
            raise ConfigError("invalid configuration: " + "; ".join(p))
        return cfg

    def owner(self, i: int) -> int:
        """The layer whose tensors layer ``i`` uses (itself unless it names another)."""
        shared = self.layers[i].weights_of
        return i if shared is None else shared

    def sizes_from_tensors(self, shapes: dict) -> None:
        """Fill in what config.json leaves to the checkpoint: the inner size of a right mixer's decay products, from the
        shape of its ``w1`` tensor (name -> shape of every tensor of the folder)."""
        layers = list(self.layers)
        for i, layer in enumerate(layers):
            if layer.type == "parallel" and layer.mixer.right.rank == 0:
                shape = shapes.get(f"l{self.owner(i)}.mix.right.w1")
                if shape is not None and len(shape) == 2:
                    right = dataclasses.replace(layer.mixer.right, rank=int(shape[0]))
                    layers[i] = dataclasses.replace(layer, mixer=dataclasses.replace(layer.mixer, right=right))
        self.layers = tuple(layers)

    def validate(self) -> list:
        p = []
        if not self.eps > 0:
            p.append("norm.eps must be positive")
        if self.width % self.norm_groups:
            p.append(f"norm.groups: a row of {self.width} numbers does not split into {self.norm_groups} equal parts")
        for i, layer in enumerate(self.layers):
            w = f"layers[{i}].mixer"
            att = layer.mixer if layer.type == "attention" else layer.mixer.left
            aw = w if layer.type == "attention" else f"{w}.left"
            if not att.scale > 0:
                p.append(f"{aw}: scale must be positive")
            if att.heads % att.kv_heads:
                p.append(f"{aw}: {att.heads} heads over {att.kv_heads} kv_heads")
            if not att.rot.base > 0:
                p.append(f"{aw}.rot: base must be positive")
            if att.rot.dims % 2 or att.rot.dims > att.dim:
                p.append(f"{aw}.rot: dims must be even and at most the head's {att.dim}, got {att.rot.dims}")
            if layer.type == "attention" and att.heads > 32:
                p.append(f"{aw}: scores are mixed over at most 32 heads")
            if layer.type == "parallel":
                if att.vdim % 2:
                    p.append(f"{aw}: values are rotated in pairs, vdim must be even, got {att.vdim}")
                if att.softcap < 0:
                    p.append(f"{aw}: softcap must be positive")
                if layer.mixer.right.dim > 256:
                    p.append(f"{w}.right: at most 256 numbers a head, got {layer.mixer.right.dim}")
            f = layer.mlp
            if f is not None and f.kind == "moe":
                if f.top > f.experts:
                    p.append(f"layers[{i}].mlp: top {f.top} of {f.experts} experts")
                if f.top > 32:
                    p.append(f"layers[{i}].mlp: at most 32 experts a token")
            j = layer.weights_of
            if j is not None:
                if not 0 <= j < len(self.layers) or j == i or self.layers[j].weights_of is not None:
                    p.append(f"layers[{i}]: 'weights_of' must name another layer that has tensors of its own, got {j}")
                elif dataclasses.replace(self._without_rank(layer), weights_of=None) != self._without_rank(self.layers[j]):
                    p.append(f"layers[{i}]: a layer that uses layer {j}'s tensors must have the same sizes and constants")
        return p

    @staticmethod
    def _without_rank(layer):
        if layer.type != "parallel":
            return layer
        return dataclasses.replace(layer, mixer=dataclasses.replace(layer.mixer, right=dataclasses.replace(layer.mixer.right, rank=0)))

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def to_dict(self) -> dict:
        out = {"architecture": self.architectures[0] if self.architectures else "Reverax",
               "layers": [layer.to_dict() for layer in self.layers], "logit_scale": self.logit_scale,
               "norm": {"eps": self.eps, "groups": self.norm_groups}, "vocab": self.vocab, "width": self.width}
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out
