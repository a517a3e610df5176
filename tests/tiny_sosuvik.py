"""Tiny Sosuvik configurations and helpers for the tests.

S1: a loop over the first two layers, three passes; an attention layer whose value heads are wider than its key heads,
rotated over half a head with scaled frequencies, capped scores, chunks of 24 (pages of 16: edges inside pages and on
their borders); a latent layer (24 + 8 numbers a page row); a layer without a feed-forward.
S2: no loop, no chunks, no cap, no scaling, whole heads rotated, as many key heads as query heads, experts without
groups, top = experts in one layer, a logit factor of 1 left out.
S3: sizes that the tensor-core kernels take (heads of 64 in groups of 4, a page row of 128 numbers, pages of 64, experts
of 128 inner numbers), a loop over the middle layer alone.
S4: sizes that are multiples of nothing much; groups of one expert; chunks shorter than a page; a loop that runs once;
two looped layers of different kinds.
"""
import json
import os

import torch


def rot(base, dims, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling:
        out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return out


def attn(heads, kv_heads, dim, vdim, rotation, scale=None, softcap=None, chunk=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rotation,
         "scale": scale if scale is not None else dim ** -0.5}
    if softcap:
        m["softcap"] = softcap
    if chunk:
        m["mask"] = {"size": chunk}
    return m


def lat(heads, dim, rot_dim, vdim, kv_rank, base=10000.0, scale=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "rot": rot(base, rot_dim),
            "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}


def moe(ff, experts, top, limit, scale=1.0, groups=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}


def layer(mixer, mlp):
    return {"type": "latent_attention" if "kv_rank" in mixer else "attention", "mixer": mixer, "mlp": mlp}


def model(vocab, width, layers, loop=None, eps=1e-6, logit_scale=None):
    out = {"architecture": "Sosuvik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    if logit_scale is not None:
        out["logit_scale"] = logit_scale
    return out


S1 = model(211, 64, [layer(attn(4, 2, 16, 24, rot(5000.0, 8, (4.0, 64, 8.0, 2.0)), softcap=5.0, chunk=24), moe(40, 6, 2, 0.4, 1.5, (3, 2))),
                     layer(lat(2, 16, 8, 12, 24), moe(24, 4, 3, 0.3, 2.0, (2, 2))),
                     layer(attn(2, 1, 8, 8, rot(100.0, 8), softcap=3.0, chunk=31), None)],
           loop=(0, 2, 3), logit_scale=0.7)
S2 = model(300, 96, [layer(attn(3, 3, 32, 32, rot(1e4, 32)), moe(48, 5, 5, 0.5)),
                     layer(lat(3, 8, 16, 16, 40, base=500.0), moe(32, 8, 1, 0.25, 0.5, (4, 1))),
                     layer(attn(6, 2, 16, 8, rot(1e6, 4), chunk=50), moe(16, 3, 2, 1.0, 3.0))], eps=1e-5)
S3 = model(352, 128, [layer(attn(8, 2, 64, 64, rot(2e5, 32, (8.0, 128, 16.0, 1.0)), softcap=30.0, chunk=130), moe(128, 6, 2, 0.6, 2.0, (3, 2))),
                      layer(lat(8, 32, 64, 32, 64, base=3e5), moe(64, 4, 2, 0.5, 1.0, (2, 1))),
                      layer(attn(4, 4, 128, 128, rot(1e4, 128), chunk=64), None)],
           loop=(1, 2, 2), logit_scale=2.0)
S4 = model(97, 90, [layer(lat(5, 6, 6, 10, 20, base=77.0), moe(20, 4, 2, 0.2, 1.3, (4, 2))),
                    layer(attn(3, 3, 10, 6, rot(300.0, 4, (2.0, 16, 4.0, 1.0)), scale=0.4, softcap=2.0, chunk=7), moe(12, 9, 3, 0.35, 2.5, (3, 1))),
                    layer(lat(2, 14, 2, 14, 18), None),
                    layer(attn(2, 1, 12, 20, rot(50.0, 12), softcap=8.0), moe(36, 2, 1, 0.5))],
           loop=(1, 3, 1), eps=1e-4, logit_scale=0.25)
CONFIGS = {"S1": (S1, 16), "S2": (S2, 32), "S3": (S3, 64), "S4": (S4, 16)}


def make_folder(tmp_path, raw: dict, seed: int = 0, sharp: float = 6.0, out_boost: float = 15.0) -> str:
    """A model folder from the engine's random-weights mode with the tensors whose useful range is not N(0, 0.02) scaled:
    queries and keys by ``sharp`` (a few keys then carry most of a row's weight, and a wrong, missing or stale key shows),
    the mixers' output projections by ``out_boost`` (what a mixer adds is then comparable to the stream), the routers so
    that scores spread over (0, 1), the corrections so that they change choices, the loop's product and step vectors so
    that the stream keeps its size through a pass."""
    from safetensors.torch import load_file, save_file
    from rust_mlx_b200.config import SosuvikConfig
    from rust_mlx_b200.weights import write_random_model
    folder = os.path.join(str(tmp_path), f"sosuvik_{abs(hash(json.dumps(raw, sort_keys=True))) % 10**8}_{seed}_{sharp}_{out_boost}")
    if not os.path.exists(os.path.join(folder, "model.safetensors")):
        write_random_model(SosuvikConfig.from_dict(raw), folder, seed=seed, store_dtype="bfloat16")
        t = load_file(os.path.join(folder, "model.safetensors"))
        factors = {".mix.q": sharp, ".mix.k": sharp, ".mix.uk": sharp, ".mix.dkv": 3.0, ".mix.o": out_boost, ".mlp.router": 40.0,
                   ".mlp.correction": 15.0, ".down": 10.0, "loop.in": 6.0, "loop.step": 25.0}
        for k in t:
            for ending, f in factors.items():
                if k.endswith(ending):
                    t[k] = (t[k].float() * f).to(torch.bfloat16).to(t[k].dtype)
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
