"""Configuration of the Sosuvik decoder.

config.json of this family is nested:

    architecture      "Sosuvik"
    vocab, width
    norm.eps          the eps of every RMS norm
    logit_scale       what the logits are multiplied with
    loop              optional: start, stop, times: layers start .. stop - 1 run `times` times in a row with the same weights
                      (every pass with caches of its own), each pass behind a product that mixes the embedding's output back in
    layers[]          one entry a layer, in order:
        type          "attention" or "latent_attention"
        mixer         attention: heads, kv_heads, dim (query/key numbers a head), vdim, scale, softcap (optional),
                          mask.size (optional: a query reads its own chunk of that many positions only),
                          rot: base, dims (numbers of a head that are rotated), scaling (optional): factor, original, fast, slow
                      latent_attention: heads, dim (numbers of a query head that meet the latent), rot_dim (rotated numbers of a
                          query head, and of the one key part all heads share), vdim, kv_rank, scale, rot: base, dims (= rot_dim)
        mlp           null, or kind "moe": expert.ff, expert.limit, router.experts, router.top, router.scale,
                      router.groups.count and .keep (optional)

Every size and constant is read from here; every problem of a file is reported in one ``ConfigError``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .base import ConfigError, ModelConfig
from .resolorn import _float, _int

MIXERS = ("attention", "latent_attention")


@dataclass(frozen=True)
class RotationConfig:
    base: float
    dims: int
    scaling: Optional[tuple] = None      # (factor, original, fast, slow) or None

    def to_dict(self) -> dict:
        out = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            factor, original, fast, slow = self.scaling
            out["scaling"] = {"factor": factor, "fast": fast, "original": original, "slow": slow}
        return out

    def scaling_dict(self) -> Optional[dict]:
        """The scaling in the words that ``parts.position.scaled_inv_freq`` reads."""
        if self.scaling is None:
            return None
        factor, original, fast, slow = self.scaling
        return {"rope_type": "yarn", "factor": factor, "original_max_position_embeddings": original, "beta_fast": fast,
                "beta_slow": slow}


@dataclass(frozen=True)
class ChunkedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotationConfig
    softcap: float = 0.0        # 0: none
    chunk: int = 0              # 0: every earlier position is read

    def to_dict(self) -> dict:
        out = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "rot": self.rot.to_dict(), "scale": self.scale,
               "vdim": self.vdim}
        if self.chunk:
            out["mask"] = {"size": self.chunk}
        if self.softcap:
            out["softcap"] = self.softcap
        return out


@dataclass(frozen=True)
class RotatedLatentConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: RotationConfig

    def to_dict(self) -> dict:
        return {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "rot": self.rot.to_dict(), "rot_dim": self.rot_dim,
                "scale": self.scale, "vdim": self.vdim}


@dataclass(frozen=True)
class GroupedExpertsConfig:
    ff: int
    limit: float
    experts: int
    top: int
    scale: float
    groups: int = 1
    keep: int = 1

    def to_dict(self) -> dict:
        router = {"experts": self.experts, "scale": self.scale, "top": self.top}
        if self.groups != 1 or self.keep != 1:
            router["groups"] = {"count": self.groups, "keep": self.keep}
        return {"expert": {"ff": self.ff, "limit": self.limit}, "kind": "moe", "router": router}


@dataclass(frozen=True)
class SosuvikLayer:
    type: str
    mixer: object
    mlp: Optional[GroupedExpertsConfig]

    def to_dict(self) -> dict:
        return {"mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp is not None else None, "type": self.type}


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int

    def to_dict(self) -> dict:
        return {"start": self.start, "stop": self.stop, "times": self.times}


def _rotation(p, where, m) -> RotationConfig:
    rot = m.get("rot")
    if not isinstance(rot, dict):
        p.append(f"{where}: missing 'rot' (an object with 'base' and 'dims')")
        return RotationConfig(10000.0, 0)
    base = _float(p, f"{where}.rot", rot, "base")
    dims = _int(p, f"{where}.rot", rot, "dims", minimum=0)
    scaling = rot.get("scaling")
    if scaling is not None:
        if not isinstance(scaling, dict):
            p.append(f"{where}.rot: 'scaling' must be an object")
            scaling = None
        else:
            w = f"{where}.rot.scaling"
            scaling = (_float(p, w, scaling, "factor"), _float(p, w, scaling, "original"), _float(p, w, scaling, "fast"),
                       _float(p, w, scaling, "slow"))
    return RotationConfig(base, dims, scaling)


@dataclass
class SosuvikConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    eps: float = 0.0
    logit_scale: float = 1.0
    layers: tuple = ()
    loop: Optional[LoopConfig] = None
    eos_token_id: tuple = ()

    @classmethod
    def from_dict(cls, raw: dict) -> "SosuvikConfig":
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
                mask = m.get("mask")
                mixer = ChunkedAttentionConfig(
                    heads=_int(p, w, m, "heads"), kv_heads=_int(p, w, m, "kv_heads"), dim=_int(p, w, m, "dim"),
                    vdim=_int(p, w, m, "vdim"), scale=_float(p, w, m, "scale"), rot=_rotation(p, w, m),
                    softcap=_float(p, w, m, "softcap", required=False, default=0.0),
                    chunk=_int(p, f"{w}.mask", mask, "size") if isinstance(mask, dict) else 0)
            else:
                mixer = RotatedLatentConfig(
                    heads=_int(p, w, m, "heads"), dim=_int(p, w, m, "dim"), rot_dim=_int(p, w, m, "rot_dim", minimum=0),
                    vdim=_int(p, w, m, "vdim"), kv_rank=_int(p, w, m, "kv_rank"), scale=_float(p, w, m, "scale"),
                    rot=_rotation(p, w, m))
            f = entry.get("mlp")
            mlp = None
            if f is not None:
                if not isinstance(f, dict) or f.get("kind") != "moe":
                    p.append(f"{where}.mlp: 'kind' must be 'moe' (or the layer's 'mlp' null)")
                else:
                    router = f.get("router") if isinstance(f.get("router"), dict) else {}
                    groups = router.get("groups")
                    mlp = GroupedExpertsConfig(
                        ff=_int(p, f"{where}.mlp.expert", f.get("expert"), "ff"), limit=_float(p, f"{where}.mlp.expert", f.get("expert"), "limit"),
                        experts=_int(p, f"{where}.mlp.router", router, "experts"), top=_int(p, f"{where}.mlp.router", router, "top"),
                        scale=_float(p, f"{where}.mlp.router", router, "scale", required=False, default=1.0),
                        groups=_int(p, f"{where}.mlp.router.groups", groups, "count") if isinstance(groups, dict) else 1,
                        keep=_int(p, f"{where}.mlp.router.groups", groups, "keep") if isinstance(groups, dict) else 1)
            layers.append(SosuvikLayer(kind, mixer, mlp))
        loop = raw.get("loop")
        if loop is not None:
            if not isinstance(loop, dict):
                p.append("config: 'loop' must be an object with 'start', 'stop' and 'times'")
                loop = None
            else:
                loop = LoopConfig(_int(p, "loop", loop, "start", minimum=0), _int(p, "loop", loop, "stop", minimum=0),
                                  _int(p, "loop", loop, "times"))
        if p:
            raise ConfigError("invalid configuration: " + "; ".join(p))
        eos = raw.get("eos_token_id")
        eos = () if eos is None else (tuple(eos) if isinstance(eos, (list, tuple)) else (eos,))
        cfg = cls(model_type="sosuvik", architectures=(name or "Sosuvik",), vocab=vocab, width=width, eps=eps,
                  logit_scale=logit_scale, layers=tuple(layers), loop=loop, eos_token_id=eos)
        cfg._raw = dict(raw)
        p = cfg.validate()
        if p:
            raise ConfigError("invalid configuration: " + "; ".join(p))
        return cfg

    def validate(self) -> list:
        p = []
        if not self.eps > 0:
            p.append("norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            m, w = layer.mixer, f"layers[{i}].mixer"
            if not m.scale > 0:
                p.append(f"{w}: scale must be positive")
            if not m.rot.base > 0:
                p.append(f"{w}.rot: base must be positive")
            if m.rot.dims % 2:
                p.append(f"{w}.rot: dims must be even, got {m.rot.dims}")
            if m.rot.scaling is not None:
                factor, original, fast, slow = m.rot.scaling
                if not (factor >= 1 and original > 0 and fast > 0 and slow > 0):
                    p.append(f"{w}.rot.scaling: factor at least 1, original, fast and slow positive")
            if layer.type == "attention":
                if m.heads % m.kv_heads:
                    p.append(f"{w}: {m.heads} heads over {m.kv_heads} kv_heads")
                if m.rot.dims > m.dim:
                    p.append(f"{w}.rot: dims {m.rot.dims} beyond the head's {m.dim}")
                if m.softcap < 0:
                    p.append(f"{w}: softcap must be positive")
            elif m.rot.dims != m.rot_dim:
                p.append(f"{w}.rot: dims {m.rot.dims} must equal rot_dim {m.rot_dim}")
            f = layer.mlp
            if f is not None:
                w = f"layers[{i}].mlp"
                if f.top > f.experts:
                    p.append(f"{w}: top {f.top} of {f.experts} experts")
                if f.top > 32:
                    p.append(f"{w}: at most 32 experts a token")
                if f.experts % f.groups or not 1 <= f.keep <= f.groups:
                    p.append(f"{w}: {f.experts} experts in {f.groups} groups of which {f.keep} are kept")
                elif f.keep * (f.experts // f.groups) < f.top:
                    p.append(f"{w}: {f.keep} groups of {f.experts // f.groups} experts cannot give {f.top}")
                if not f.limit > 0:
                    p.append(f"{w}.expert: limit must be positive")
        if self.loop is not None:
            lp = self.loop
            if not 0 <= lp.start < lp.stop <= len(self.layers):
                p.append(f"loop: layers {lp.start} .. {lp.stop - 1} of {len(self.layers)}")
        return p

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def to_dict(self) -> dict:
        out = {"architecture": self.architectures[0] if self.architectures else "Sosuvik",
               "layers": [layer.to_dict() for layer in self.layers], "logit_scale": self.logit_scale,
               "norm": {"eps": self.eps}, "vocab": self.vocab, "width": self.width}
        if self.loop is not None:
            out["loop"] = self.loop.to_dict()
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out
