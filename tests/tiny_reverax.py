"""Tiny Reverax configurations and helpers for the tests.

R1: talking-heads attention with fewer key heads than query heads and part of a head rotated; a parallel layer whose left
value heads are wider than its key heads, with a window shorter than a page, a cap, and three norm groups; a layer that
uses the parallel layer's tensors; a dense and a routed feed-forward (top 2) and a layer without one.
R2: one norm group, a logit factor of 1 left out, no cap, no window in one parallel layer and a window of 1 in another, whole
heads rotated, top = experts, one expert of one, as many key heads as query heads, a talking layer that uses another's tensors.
R3: sizes the tensor-core kernels take (left heads of 64 in a group of 4, pages of 64, experts of 128 inner numbers, state
heads of 64), a window that crosses pages, no rotation at all in the talking layer.
R4: sizes that are multiples of nothing much; one head everywhere; windows of 2 and 17; five norm groups.
"""
import json
import os

import torch


def rot(base, dims):
    return {"base": base, "dims": dims}


def talk(heads, kv_heads, dim, vdim, rotation, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rotation,
            "scale": scale if scale is not None else dim ** -0.5}


def side(left_heads, kv_heads, dim, vdim, rotation, window, softcap, right_heads, right_dim, rank, left_scale=1.0, right_scale=1.0,
         scale=None):
    left = talk(left_heads, kv_heads, dim, vdim, rotation, scale)
    if window:
        left["mask"] = {"size": window}
    if softcap:
        left["softcap"] = softcap
    return {"left": left, "right": {"heads": right_heads, "dim": right_dim, "rank": rank}, "left_scale": left_scale,
            "right_scale": right_scale}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def layer(mixer, mlp, weights_of=None):
    out = {"type": "parallel" if "left" in mixer else "attention", "mixer": mixer, "mlp": mlp}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def model(vocab, width, layers, eps=1e-5, groups=None, logit_scale=None):
    out = {"architecture": "Reverax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if groups is not None:
        out["norm"]["groups"] = groups
    if logit_scale is not None:
        out["logit_scale"] = logit_scale
    return out


_P1 = side(4, 2, 16, 24, rot(5000.0, 8), 11, 6.0, 3, 16, 5, 1.3, 0.8)
R1 = model(211, 72, [layer(talk(6, 2, 16, 8, rot(300.0, 8)), dense(40)),
                     layer(_P1, moe(24, 6, 2)),
                     layer(_P1, moe(24, 6, 2), weights_of=1),
                     layer(talk(3, 3, 8, 12, rot(1e4, 8)), None)], groups=3, logit_scale=0.7)
_T2 = talk(4, 4, 8, 8, rot(1e5, 8), scale=0.5)
R2 = model(300, 96, [layer(side(2, 2, 32, 32, rot(1e4, 32), 0, 0.0, 2, 24, 3), moe(32, 4, 4)),
                     layer(_T2, moe(16, 1, 1)),
                     layer(_T2, moe(16, 1, 1), weights_of=1),
                     layer(side(3, 1, 8, 8, rot(50.0, 4), 1, 2.0, 6, 8, 2, 0.5, 2.0), dense(20))], eps=1e-6)
R3 = model(352, 128, [layer(side(8, 2, 64, 64, rot(2e5, 32), 100, 25.0, 2, 64, 12, 1.3, 0.9), moe(128, 8, 2)),
                      layer(talk(8, 4, 32, 32, rot(1e4, 0)), dense(256)),
                      layer(side(4, 4, 32, 64, rot(1e4, 32), 70, 0.0, 4, 32, 8), None)], groups=4, logit_scale=1.5)
R4 = model(97, 90, [layer(side(1, 1, 10, 6, rot(77.0, 4), 2, 3.0, 1, 14, 1, 0.9, 1.4, scale=0.4), moe(12, 9, 3)),
                    layer(talk(1, 1, 12, 20, rot(300.0, 12)), moe(20, 2, 1)),
                    layer(side(2, 1, 6, 10, rot(900.0, 6), 17, 0.0, 5, 6, 7), dense(36))], eps=1e-4, groups=5, logit_scale=0.25)
CONFIGS = {"R1": (R1, 16), "R2": (R2, 32), "R3": (R3, 64), "R4": (R4, 16)}


def make_folder(tmp_path, raw: dict, seed: int = 0, sharp: float = 6.0, out_boost: float = 15.0) -> str:
    """A model folder from the engine's random-weights mode with the tensors whose useful range is not N(0, 0.02) scaled or
    drawn anew: queries and keys by ``sharp`` (a few keys then carry most of a row's weight, and a wrong, missing or stale key
    shows; where q and k are normed the norm weights carry the factor instead), the output projections by ``out_boost``, the
    routers so that scores spread over (0, 1), the mixing matrix of the talking heads near the identity with large
    off-diagonal numbers, sinks of both signs, decays between fast and slow, token-shift mixes in (0, 1), bonuses of size 1."""
    from safetensors.torch import load_file, save_file
    from rust_mlx_b200.config import ReveraxConfig
    from rust_mlx_b200.weights import write_random_model
    folder = os.path.join(str(tmp_path), f"reverax_{abs(hash(json.dumps(raw, sort_keys=True))) % 10**8}_{seed}_{sharp}_{out_boost}")
    if not os.path.exists(os.path.join(folder, "model.safetensors")):
        write_random_model(ReveraxConfig.from_dict(raw), folder, seed=seed, store_dtype="bfloat16")
        t = load_file(os.path.join(folder, "model.safetensors"))
        g = torch.Generator().manual_seed(seed + 17)
        factors = {".mix.q": sharp, ".mix.k": sharp, ".left.q.norm": sharp ** 0.5, ".left.k.norm": sharp ** 0.5, ".left.v": 4.0, ".mix.v": 4.0,
                   ".o": out_boost, ".down": 10.0, ".right.k": 6.0, ".right.v": 6.0, ".right.r": 6.0, ".right.g": 30.0,
                   ".right.w1": 20.0, ".right.w2": 20.0, ".q.b": 10.0, ".k.b": 10.0, ".v.b": 10.0}
        factors[".mlp.router"] = 75.0 / raw["width"] ** 0.5       # logits of size 1.5 from normed rows: scores spread, none saturates
        for k in t:
            for ending, f in factors.items():
                if k.endswith(ending):
                    t[k] = (t[k].float() * f).to(torch.bfloat16)
            shape = t[k].shape
            if k.endswith(".talk"):
                t[k] = (torch.eye(shape[0]) + 0.4 * torch.randn(shape, generator=g)).to(torch.bfloat16)
            elif k.endswith(".sink"):
                t[k] = (2.0 * torch.randn(shape, generator=g)).to(torch.bfloat16)
            elif k.endswith(".w0"):
                t[k] = (torch.rand(shape, generator=g) * 5.0 - 4.5).to(torch.bfloat16)      # decays from 0.99 down to 0.2
            elif ".right.mu." in k:
                t[k] = torch.rand(shape, generator=g).to(torch.bfloat16)
            elif k.endswith(".right.u"):
                t[k] = torch.randn(shape, generator=g).to(torch.bfloat16)
            elif k.endswith(".ls1") or k.endswith(".ls2"):
                t[k] = (0.5 + torch.rand(shape, generator=g)).to(torch.bfloat16)
        save_file(t, os.path.join(folder, "model.safetensors"))
    return folder


def weights(folder: str) -> dict:
    from safetensors.torch import load_file
    return {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}


def row_error(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per row: root mean square of the difference (means taken off) over that of the wanted row."""
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-12)
