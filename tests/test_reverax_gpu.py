"""Reverax on the GPU against its plain implementation (tests/plain_reverax.py): every mechanism alone, then whole models
replayed in every way of cutting, in both dtypes, through the engine's step function, scheduler and command line."""
import math
import random

import pytest
import torch

import plain_reverax as plain
import replay
import tiny
import tiny_reverax as tr
from test_kernels_gpu import _Batch, paged_setup

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
F = torch.float64
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


def ops():
    from rust_mlx_b200.kernels import ops as o
    return o


def rnd(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


def close(got, want, dtype, what=""):
    got, want = got.double().cpu(), want.double()
    err = (got - want).abs() / (1.0 + want.abs())
    assert not torch.isnan(got).any(), what
    assert err.max().item() < TOL[dtype], (what, err.max().item())


def context(dtype=torch.float32):
    from rust_mlx_b200.engine.workspace import Workspace
    from rust_mlx_b200.parts import BuildContext
    return BuildContext(DEV, dtype, ops().default, Workspace(DEV))


def bind(part, seed=0, dtype=torch.float32, scale=None, draw=None):
    """Random tensors for ``part`` (``scale``: name ending -> factor; ``draw``: name ending -> function of a shape), bound;
    returns them in float64 on the host."""
    from rust_mlx_b200.weights.random_init import random_tensors
    tensors = random_tensors(part.all_param_specs(), seed, dtype, DEV)
    for k in tensors:
        for ending, factor in (scale or {}).items():
            if k.endswith(ending):
                tensors[k] = (tensors[k].float() * factor).to(tensors[k].dtype)
        for ending, fn in (draw or {}).items():
            if k.endswith(ending) or ending in k:
                tensors[k] = fn(tuple(tensors[k].shape)).to(device=DEV, dtype=tensors[k].dtype)
    host = {k: v.detach().cpu().to(F) for k, v in tensors.items()}
    part.bind_all(tensors, context(dtype))
    return host


# ------------------------------------------------------------------------------------------------ kernels alone

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows, width, groups", [(1, 64, 1), (37, 90, 3), (300, 336, 2), (5, 4096, 8), (2, 6, 6), (9, 1280, 64), (3, 35, 5)])
def test_the_streams_add_and_norm_in_groups(dtype, rows, width, groups):
    """v = h + va * (m1 d1 + m2 d2) + vb * d3, normed in groups with two weights; every term and vector may be missing; the
    gathered form leaves h alone."""
    dt = DT[dtype]
    h0 = rnd((rows, width), 1, 3.0)
    d = [rnd((rows, width), 2 + i).to(dt) for i in range(3)]
    va, vb, w, w2 = (rnd((width,), 7 + i).abs() + 0.3 for i in range(4))
    for use in ((1, 1, 1, 1, 1), (1, 0, 1, 1, 0), (1, 1, 0, 0, 1), (0, 0, 1, 0, 1), (0, 0, 0, 0, 0), (1, 0, 0, 1, 1)):
        d1, d2, d3 = (d[i] if use[i] else None for i in range(3))
        a, b = (va if use[3] else None), (vb if use[4] else None)
        v = h0.double()
        if d1 is not None:
            inner = 1.3 * d1.double() + (0.6 * d2.double() if d2 is not None else 0)
            v = v + (a.double() * inner if a is not None else inner)
        if d3 is not None:
            v = v + (b.double() * d3.double() if b is not None else d3.double())
        normed = plain.rms(v.reshape(rows, groups, width // groups), 1e-5).reshape(rows, width)
        h = h0.clone().to(DEV)
        x, x2 = torch.empty(rows, width, dtype=dt, device=DEV), torch.empty(rows, width, dtype=dt, device=DEV)
        dev = lambda t: None if t is None else t.to(DEV)      # noqa: E731
        terms = (dev(d1), dev(d2), dev(d3), 1.3, 0.6, dev(a), dev(b))
        ops().add_group_rmsnorm(h, terms, w.to(DEV), 1e-5, groups, x, weight2=w2.to(DEV), x2_out=x2)
        close(h, v, "float32", ("h", use))
        close(x, normed * w.double(), dtype, ("x", use))
        close(x2, normed * w2.double(), dtype, ("x2", use))
        pick = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
        h = h0.clone().to(DEV)
        xr = torch.empty(2, width, dtype=dt, device=DEV)
        ops().add_group_rmsnorm(h, terms, w.to(DEV), 1e-5, groups, xr, rows=pick)
        assert torch.equal(h.cpu(), h0)
        assert torch.equal(xr.cpu(), x[pick.long()].cpu())


def split_rows(proj, bias, qn, kn, eps, pos, nq, nkv, dq, dv, base, rot, near, turn_values):
    """What the split kernel should give for rows [q | k | v]: q [T, nq, dq], k [T, nkv, dq], v [T, nkv, dv] in float64."""
    t = proj.shape[0]
    x = proj.double() + (bias.double() if bias is not None else 0)
    q, k, v = x[:, :nq * dq].reshape(t, nq, dq), x[:, nq * dq:(nq + nkv) * dq].reshape(t, nkv, dq), x[:, (nq + nkv) * dq:].reshape(t, nkv, dv)
    if qn is not None:
        q, k = plain.rms(q, eps) * qn.double(), plain.rms(k, eps) * kn.double()
    q, k = plain.turn(q, pos, base, rot, near), plain.turn(k, pos, base, rot, near)
    if turn_values:
        v = plain.turn(v, pos, base, dv, near)
    return q, k, v


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq, nkv, dq, dv, hd, rot, near, normed, biased, turn_values, page", [
    (4, 2, 16, 24, 32, 8, False, True, True, True, 4), (6, 2, 16, 8, 16, 8, True, False, True, False, 16), (3, 3, 8, 12, 12, 0, True, False, False, False, 8),
    (8, 2, 64, 64, 64, 32, False, True, True, True, 64), (1, 1, 10, 6, 16, 4, False, True, False, True, 2), (2, 1, 48, 48, 64, 48, True, False, True, True, 16),
    (5, 5, 40, 96, 96, 40, False, True, True, True, 32)])
def test_projection_rows_split_normed_rotated_and_written(dtype, nq, nkv, dq, dv, hd, rot, near, normed, biased, turn_values, page):
    """Every option of the general split kernel; pools hold NaN wherever nothing is written; heads are padded with zeros; a second
    call with write_kv off writes q alone.  Then the results are turned back by the rows' own positions."""
    dt = DT[dtype]
    lengths, new = [21, 7, 40], [9, 1, 40]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    batch = _Batch(lengths, new, status)
    k_pool, v_pool, table, _, _ = paged_setup(lengths, nkv, hd, page, dt, seed=3)
    k_pool.fill_(float("nan"))
    v_pool.fill_(float("nan"))
    n = sum(new)
    proj = rnd((n, (nq + nkv) * dq + nkv * dv), 5).to(dt)
    bias = rnd((proj.shape[1],), 6) if biased else None
    qn, kn = (rnd((dq,), 7).abs() + 0.5, rnd((dq,), 8).abs() + 0.5) if normed else (None, None)
    base = 700.0
    pos = batch.positions.cpu()
    want_q, want_k, want_v = split_rows(proj, bias, qn, kn, 1e-5, pos, nq, nkv, dq, dv, base, rot, near, turn_values)

    def table_of(dims):
        if dims == 0:
            return None
        f = (base ** (-2.0 * torch.arange(dims // 2, dtype=F) / dims)).float().to(DEV)
        out = torch.empty(n, dims, dtype=torch.float32, device=DEV)
        ops().rope_table(batch.positions, f, dims, out)
        return out
    cs, vcs = table_of(rot), (table_of(dv) if turn_values else None)
    dev = lambda t: None if t is None else t.to(DEV)      # noqa: E731
    q = torch.full((n, nq * hd), float("nan"), dtype=dt, device=DEV)
    ops().heads_rope_cache(proj.to(DEV), dev(bias), dev(qn), dev(kn), 1e-5, cs, rot, near, vcs, near, batch.positions, batch.seq_index, table,
                           page, k_pool, v_pool, q, nq, nkv, dq, dv, hd, True, status)
    assert status.item() == 0
    got_q = q.view(n, nq, hd).cpu()
    close(got_q[..., :dq], want_q, dtype, "q")
    assert (got_q[..., dq:] == 0).all()
    seq, written = batch.seq_index.cpu(), torch.zeros_like(k_pool[..., 0].cpu(), dtype=torch.bool)
    for t in range(n):
        p = int(pos[t])
        pg = int(table[seq[t], p // page])
        close(k_pool[pg, :, p % page, :dq], want_k[t], dtype, "k")
        close(v_pool[pg, :, p % page, :dv], want_v[t], dtype, "v")
        assert (k_pool[pg, :, p % page, dq:] == 0).all() and (v_pool[pg, :, p % page, dv:] == 0).all()
        written[pg, :, p % page] = True
    assert torch.isnan(k_pool.cpu()[~written]).all() and torch.isnan(v_pool.cpu()[~written]).all()
    before = k_pool.clone()
    q2 = torch.empty_like(q)
    ops().heads_rope_cache(proj.to(DEV), dev(bias), dev(qn), dev(kn), 1e-5, cs, rot, near, vcs, near, batch.positions, batch.seq_index, table,
                           page, k_pool, v_pool, q2, nq, nkv, dq, dv, hd, False, status)
    assert torch.equal(q2, q) and torch.equal(k_pool.nan_to_num(7.0), before.nan_to_num(7.0))
    if dv % 2 == 0:
        # turning back: rows of nq heads, hd apart, by minus the rows' angles, into dense rows
        o = torch.zeros(n, nq, hd, dtype=dt)
        o[..., :dv] = rnd((n, nq, dv), 9).to(dt)
        back = torch.empty(n, nq * dv, dtype=dt, device=DEV)
        ops().unrotate_heads(o.view(n, nq * hd).to(DEV), table_of(dv), near, back, nq, dv, hd)
        close(back.view(n, nq, dv), plain.turn(o[..., :dv].double(), pos, base, dv, near, sign=-1.0), dtype, "turned back")


def talking_rows(q, k, v, talk, qpos, window, scale):
    """q [T, H, d] at positions qpos, k [S, G, d], v [S, G, dv] for positions 0 .. S - 1: the mixed-score attention in float64."""
    t, H, _ = q.shape
    kv_of = torch.arange(H) // (H // k.shape[1])
    s = torch.einsum("ihc,jhc->hij", q.double(), k.double()[:, kv_of]) * scale
    s = torch.einsum("hg,gij->hij", talk.double(), s)
    j = torch.arange(k.shape[0])
    ok = j[None, :] <= qpos[:, None]
    if window:
        ok &= j[None, :] > qpos[:, None] - window
    a = torch.softmax(s.masked_fill(~ok, -math.inf), dim=-1)
    return torch.einsum("hij,jhc->ihc", a, v.double()[:, kv_of])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq, nkv, hd, dq, dv, page, window", [(4, 2, 16, 16, 16, 16, 0), (6, 2, 16, 16, 8, 8, 0), (3, 3, 12, 8, 12, 4, 21), (6, 6, 48, 48, 48, 64, 0),
                                                              (1, 1, 20, 12, 20, 16, 0), (8, 4, 32, 32, 32, 32, 50), (16, 2, 64, 64, 64, 64, 0),
                                                              (16, 16, 128, 128, 128, 64, 0),       # (key rows so wide that a block takes 16 keys at a time)
                                                              (24, 8, 16, 16, 16, 16, 0), (32, 32, 32, 32, 32, 32, 7)])
@pytest.mark.parametrize("portions", [True, False])
def test_attention_with_scores_mixed_over_the_heads(dtype, nq, nkv, hd, dq, dv, page, window, portions):
    """Portions of several sequences beside single decoded tokens (in bfloat16: the tensor-core kernel where it takes the head
    size), or decoded tokens alone (in bfloat16: keys split over blocks and merged); NaN in every slot of the pools that must not be read; the
    mixing matrix far from the identity, so that a head's row depends on every other head's scores."""
    dt = DT[dtype]
    lengths, new = ([150, 37, 260, 1, 64], [150, 1, 45, 1, 1]) if portions else ([700, 37, 260, 1, 1500], [1, 1, 1, 1, 1])
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    batch = _Batch(lengths, new, status)
    k_pool, v_pool, table, ks, vs = paged_setup(lengths, nkv, hd, page, dt, seed=nq)
    talk = torch.eye(nq) + 0.5 * rnd((nq, nq), 4)
    n = sum(new)
    q = rnd((n, nq, hd), 5).to(dt)
    out = torch.empty(n, nq * dv, dtype=dt, device=DEV)
    ops().default.attention_talk(q.view(n, nq * hd).to(DEV), k_pool, v_pool, talk.to(DEV), batch, table, page, out, nq, nkv, hd, dq, dv, window,
                                 0.3, None)
    assert status.item() == 0
    at = 0
    for s, (length, c) in enumerate(zip(lengths, new)):
        qpos = torch.arange(length - c, length)
        want = talking_rows(q[at:at + c, :, :dq], ks[s][..., :dq], vs[s][..., :dv], talk, qpos, window, 0.3)
        close(out[at:at + c].view(c, nq, dv), want, dtype, (s, length, c))
        at += c


@pytest.mark.parametrize("splits", [1, 2, 3, 5])
@pytest.mark.parametrize("nq, nkv, hd, dv, window", [(4, 2, 16, 16, 0), (16, 4, 64, 64, 0), (6, 3, 48, 40, 90), (8, 8, 128, 128, 0)])
def test_tensor_core_mixed_score_attention_with_and_without_key_splits(nq, nkv, hd, dv, window, splits):
    """The tensor-core kernel called as it is, with tiles of up to 16 tokens whose keys go to 1, 2, 3 or 5 blocks (more blocks than
    some tiles have key tiles: their shares are empty)."""
    dt, page = torch.bfloat16, 32
    lengths, new = [150, 37, 260, 1, 64, 300], [150, 1, 45, 1, 17, 2]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    batch = _Batch(lengths, new, status)
    k_pool, v_pool, table, ks, vs = paged_setup(lengths, nkv, hd, page, dt, seed=nq)
    talk = torch.eye(nq) + 0.5 * rnd((nq, nq), 4)
    n = sum(new)
    q = rnd((n, nq, hd), 5).to(dt)
    out = torch.full((n, nq * dv), float("nan"), dtype=dt, device=DEV)
    ops().attention_talk_mma(q.view(n, nq * hd).to(DEV), k_pool, v_pool, talk.to(DEV), batch, table, page, out, nq, nkv, hd, dv, window, 0.3, splits)
    assert status.item() == 0
    at = 0
    for s, (length, c) in enumerate(zip(lengths, new)):
        want = talking_rows(q[at:at + c], ks[s], vs[s][..., :dv], talk, torch.arange(length - c, length), window, 0.3)
        close(out[at:at + c].view(c, nq, dv), want, "bfloat16", (s, length, c))
        at += c


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_single_far_key_decides_under_mixed_scores(dtype):
    """One key among 700 is made to stand out for ONE head; through the mixing matrix it decides other heads' rows too, with
    the sign and size that the matrix gives; prompt rows and decoded rows."""
    dt = DT[dtype]
    nq, nkv, hd, page = 4, 2, 16, 16
    lengths, new = [700, 700], [30, 1]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    batch = _Batch(lengths, new, status)
    k_pool, v_pool, table, ks, vs = paged_setup(lengths, nkv, hd, page, dt, seed=2)
    far = 17
    talk = torch.tensor([[1.0, 0.0, 0.0, 0.0], [2.0, 1.0, 0.0, 0.0], [0.0, 0.0, 1.0, 0.0], [-3.0, 0.0, 0.0, 1.0]])
    q = rnd((sum(new), nq, hd), 3).to(dt)
    for s in range(2):
        ks[s][far, 0] = 0
        ks[s][far, 0, 3] = 40.0
        pg = int(table[s, far // page])
        k_pool[pg, 0, far % page] = ks[s][far, 0].to(DEV)
    q[:, 0, 3] = 6.0                       # head 0's score of the far key is 240 * scale
    out = torch.empty(sum(new), nq * hd, dtype=dt, device=DEV)
    ops().default.attention_talk(q.view(-1, nq * hd).to(DEV), k_pool, v_pool, talk.to(DEV), batch, table, page, out, nq, nkv, hd, hd, hd, 0, 0.25, None)
    got = out.view(-1, nq, hd).double().cpu()
    for row, s in ((0, 0), (29, 0), (30, 1)):
        v_far = vs[s][far].double()
        assert (got[row, 0] - v_far[0]).abs().max() < 0.05           # head 0 reads the far key
        assert (got[row, 1] - v_far[0]).abs().max() < 0.05           # head 1 (the same value head) is carried along by 2 x
        assert (got[row, 3] - v_far[1]).abs().max() > 0.3            # head 3 is pushed AWAY from it by -3 x
    at = 0
    for s, (length, c) in enumerate(zip(lengths, new)):
        want = talking_rows(q[at:at + c], ks[s], vs[s], talk, torch.arange(length - c, length), 0, 0.25)
        close(out[at:at + c].view(c, nq, hd), want, dtype, s)
        at += c


class _Steps:
    """A part alone with caches of its own, fed rows in portions; requests may share steps."""

    def __init__(self, part, page, dtype, max_tokens, slots=3):
        from rust_mlx_b200.cache import CachePools
        self.part, self.specs = part, part.cache_specs()
        self.pools = CachePools(dict(enumerate(self.specs)), max_tokens=max_tokens, page_size=page, max_requests=slots, dtype=dtype, device=DEV)
        for grp in self.pools.paged_groups:
            grp.k_pool.fill_(float("nan"))
            if grp.v_pool is not None:
                grp.v_pool.fill_(float("nan"))
        self.status = torch.zeros(1, dtype=torch.int32, device=DEV)
        self.at = {}

    def step(self, rows: dict):
        """rows: request -> [c, width] tensor; returns request -> output rows."""
        from rust_mlx_b200.engine.batch import SequenceInput, build_batch
        seqs = []
        for rid, x in rows.items():
            if rid not in self.at:
                self.pools.open(rid)
                self.at[rid] = 0
            self.pools.table.reserve(rid, self.at[rid] + x.shape[0])
            seqs.append(SequenceInput(rid, self.at[rid], [0] * x.shape[0], []))
        batch = build_batch(seqs, self.pools, DEV, self.status, 10)
        views = tuple(self.pools.view(i, batch, False) for i in range(len(self.specs)))
        x = torch.cat(list(rows.values())).contiguous()
        y = self.part.forward(x, batch, views[0] if len(views) == 1 else views)
        if not isinstance(y, torch.Tensor):
            raise TypeError("a part alone gives a tensor")
        y = y.clone()
        out, at = {}, 0
        for rid, x in rows.items():
            out[rid] = y[at:at + x.shape[0]]
            at += x.shape[0]
            self.at[rid] += x.shape[0]
            self.pools.table.commit(rid, self.at[rid])
        assert self.status.item() == 0
        return out

    def close(self, rid):
        self.pools.table.close(rid)
        del self.at[rid]


def in_portions(part, x, cuts, page, dtype=torch.float32):
    run = _Steps(part, page, dtype, -(-x.shape[0] // page) * page + 2 * page)
    outs, at = [], 0
    for c in cuts:
        outs.append(run.step({5: x[at:at + c]})[5])
        at += c
    assert at == x.shape[0]
    return torch.cat(outs)


CUTS = (11, 1, 2, 1, 1, 7, 1, 1, 2, 19, 1, 3, 2, 40, 1, 1)


@pytest.mark.parametrize("heads, kv_heads, dim, vdim, dims, page", [(6, 2, 16, 8, 8, 4), (3, 3, 8, 12, 8, 8), (6, 3, 48, 48, 48, 16), (1, 1, 12, 20, 0, 16),
                                                                  (4, 1, 32, 32, 16, 64)])
def test_talking_attention_part_over_steps(heads, kv_heads, dim, vdim, dims, page):
    from rust_mlx_b200.parts.attention import TalkingAttentionMixer
    from rust_mlx_b200.parts.position import RotaryEmbedding
    width = 40
    mixer = TalkingAttentionMixer("m", width, heads, kv_heads, dim, vdim, RotaryEmbedding(dim, 777.0, rotary_dim=dims, interleaved=True), 0.3, bias=True)
    w = bind(mixer, seed=heads, scale={".q": 25.0, ".k": 25.0, ".v": 20.0, ".b": 30.0},
             draw={".talk": lambda s: torch.eye(s[0]) + 0.5 * rnd(s, 1)})
    x = rnd((sum(CUTS), width), 3).to(DEV)
    got = in_portions(mixer, x, CUTS, page)
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": tr.rot(777.0, dims), "scale": 0.3}
    want = plain.talking_attention(x.double().cpu(), w, "m", m, False)
    assert tiny.max_abs(got.cpu(), want) < 3e-5 * (1 + want.abs().max().item())


@pytest.mark.parametrize("heads, kv_heads, dim, vdim, dims, cap, window, page", [
    (4, 2, 16, 24, 8, 5.0, 11, 4), (3, 3, 8, 8, 8, 0.0, 0, 8), (6, 2, 16, 8, 4, 3.0, 5, 16), (2, 1, 12, 20, 12, 0.0, 16, 16), (1, 1, 16, 8, 8, 0.0, 1, 8),
    (4, 2, 96, 80, 32, 20.0, 33, 16), (8, 2, 64, 64, 32, 0.0, 64, 64)])
def test_windowed_attention_part_with_turned_values_and_learned_sinks_over_steps(heads, kv_heads, dim, vdim, dims, cap, window, page):
    from rust_mlx_b200.parts.attention import GatedAttentionMixer
    from rust_mlx_b200.parts.position import RotaryEmbedding
    width = 40
    mixer = GatedAttentionMixer("m", width, heads, kv_heads, dim, vdim, RotaryEmbedding(dim, 777.0, rotary_dim=dims), 0.3, sink="learned",
                                window=window, softcap=cap, bias=True, head_norm_eps=1e-5,
                                value_position=RotaryEmbedding(vdim, 777.0, rotary_dim=vdim), head_pad=True)
    w = bind(mixer, seed=heads, scale={".q.norm": 4.0, ".k.norm": 4.0, ".v": 20.0, ".b": 30.0}, draw={".sink": lambda s: 2.0 * rnd(s, 2)})
    x = rnd((sum(CUTS), width), 3).to(DEV)
    got = in_portions(mixer, x, CUTS, page)
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": tr.rot(777.0, dims), "scale": 0.3}
    if cap:
        m["softcap"] = cap
    if window:
        m["mask"] = {"size": window}
    want = plain.windowed_attention(x.double().cpu(), w, "m", m, 1e-5, False)
    assert tiny.max_abs(got.cpu(), want) < 3e-5 * (1 + want.abs().max().item())
    # the sink takes its share: without it the rows differ (shown where heads are small: the scores of large heads with these
    # weights leave a sink of size 2 no share worth the name)
    if dim <= 16:
        w0 = dict(w)
        w0["m.sink"] = torch.full_like(w["m.sink"], -50.0)
        assert tiny.max_abs(plain.windowed_attention(x.double().cpu(), w0, "m", m, 1e-5, False), want) > 1e-3 * want.abs().max().item()


def decay_draws(seed):
    return {".w0": lambda s: torch.rand(s, generator=torch.Generator().manual_seed(seed)) * 5.0 - 4.5,
            ".mu.": lambda s: torch.rand(s, generator=torch.Generator().manual_seed(seed + 1)),
            ".u": lambda s: rnd(s, seed + 2)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, dim, rank, width", [(3, 16, 5, 40), (1, 14, 1, 22), (4, 64, 16, 256), (2, 24, 3, 96), (5, 6, 7, 30), (2, 100, 4, 64), (1, 200, 2, 48)])
def test_decaying_linear_attention_part_over_steps(dtype, heads, dim, rank, width):
    """Portions down to one token; two requests that share steps and slots that are not the sequences' numbers; the state
    after the last step against the plain recurrence's."""
    from rust_mlx_b200.parts.recurrent import DecayLinearMixer
    dt = DT[dtype]
    mixer = DecayLinearMixer("m", width, heads, dim, rank, 1e-5)
    w = bind(mixer, seed=heads, dtype=dt, scale={".r": 8.0, ".k": 8.0, ".v": 8.0, ".g": 30.0, ".w1": 20.0, ".w2": 20.0}, draw=decay_draws(heads))
    xa, xb = rnd((sum(CUTS), width), 3).to(dt), rnd((70, width), 4).to(dt)
    run = _Steps(mixer, 16, dt, 256, slots=3)
    run.step({9: rnd((3, width), 8).to(dt).to(DEV)})          # a request that leaves: its slot holds a state when the next one opens
    run.close(9)
    got_a, got_b, at, bt = [], [], 0, 0
    for i, c in enumerate(CUTS):
        rows = {2: xa[at:at + c].to(DEV)}
        at += c
        if i % 2 == 1 and bt < 70:
            n = min(70 - bt, 1 + 9 * (i % 3))
            rows = {7: xb[bt:bt + n].to(DEV), **rows}
            bt += n
        out = run.step(rows)
        got_a.append(out[2])
        if 7 in out:
            got_b.append(out[7])
    assert bt == 70
    bf = dtype == "bfloat16"
    for got, x, rid in ((got_a, xa, 2), (got_b, xb, 7)):
        states = []
        want = plain.time_mix(x.double(), w, "m", {"heads": heads, "dim": dim}, 1e-5, bf, state_out=states)
        got = torch.cat(got).double().cpu()
        bound = 0.05 if bf else 3e-5
        assert (got - want).abs().max().item() < bound * (1 + want.abs().max().item()), rid
        slot = run.pools.table.slot(rid) if hasattr(run.pools.table, "slot") else None
        if slot is not None and not bf:
            state = run.pools.groups[run.pools._where[1][0]].state[run.pools._where[1][1]][slot].double().cpu()     # [heads, V, K]
            assert (state.transpose(1, 2) - states[0]).abs().max().item() < 1e-4 * (1 + states[0].abs().max().item())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts, top, inner, rows, width", [(6, 2, 40, 37, 48), (8, 3, 72, 300, 64), (4, 4, 64, 5, 40), (5, 1, 128, 64, 128), (1, 1, 16, 9, 24),
                                                             (16, 1, 64, 700, 256)])
def test_routed_part_whose_experts_read_the_weighted_row(dtype, experts, top, inner, rows, width):
    from rust_mlx_b200.parts.routed import RoutedFeedForward
    dt = DT[dtype]
    part = RoutedFeedForward("f", width, inner, experts, top, activation="relu2", names=("up", "down"), scoring="sigmoid", normalize=False,
                             gated=False, weight_input=True)
    w = bind(part, seed=experts, dtype=dt, scale={".router": 75.0 / math.sqrt(width), ".up": 10.0, ".down": 10.0})     # logits of size 1.5
    x = rnd((rows, width), 2).to(dt)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)

    class B:
        pass
    B.status = status
    got = part.forward(x.to(DEV), B).double().cpu()
    assert status.item() == 0
    bf = dtype == "bfloat16"
    margins = []
    want = plain.squared_relu_experts(x.double(), w, "f", {"router": {"experts": experts, "top": top}}, bf, margins)
    clear = margins[0] > (0.02 if bf else 1e-5)
    err = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-9)       # a row's error over the row's size
    assert clear.float().mean() > 0.6 and err[clear].max().item() < (0.03 if bf else 3e-5)
    if not bf:
        # a row alone gives the bits it gives in the batch
        one = part.forward(x[3:4].to(DEV), B).double().cpu() if rows > 3 else None
        assert one is None or torch.equal(one[0], got[3])


def test_router_gives_raw_sigmoid_scores():
    n, e, top = 50, 12, 3
    x, wr = rnd((n, 32), 1).to(DEV), rnd((e, 32), 2, 0.3).to(DEV)
    ids = torch.empty(n, top, dtype=torch.int32, device=DEV)
    wt = torch.empty(n, top, dtype=torch.float32, device=DEV)
    ops().moe_route(x, wr, top, ids, wt, scoring="sigmoid", normalize=False)
    s = torch.sigmoid(x.double().cpu() @ wr.double().cpu().T)
    best, where = torch.sort(s, dim=-1, descending=True, stable=True)
    assert torch.equal(ids.cpu().long(), where[:, :top])
    assert (wt.double().cpu() - best[:, :top]).abs().max().item() < 1e-6


@pytest.mark.parametrize("rows, top, experts, inner, k", [(3, 2, 8, 128, 64), (64, 4, 6, 64, 200), (700, 2, 3, 192, 96)])
def test_experts_up_product_squares_its_relu_in_the_epilogue(rows, top, experts, inner, k):
    g = torch.Generator().manual_seed(rows)
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(rows)]).to(torch.int32).to(DEV)
    offsets = torch.empty(experts + 1, dtype=torch.int32, device=DEV)
    pairs, where = torch.empty(rows * top, dtype=torch.int32, device=DEV), torch.empty(rows * top, dtype=torch.int32, device=DEV)
    ops().moe_sort(ids, experts, offsets, pairs, where)
    x = rnd((rows, k), 1).to(torch.bfloat16).to(DEV)
    weights = torch.rand(rows, top, generator=g).to(DEV)
    a = torch.empty(rows * top, k, dtype=torch.bfloat16, device=DEV)
    ops().moe_gather_scaled(x, pairs, weights, top, a)
    src = pairs.long().cpu()
    want_a = (weights.cpu().reshape(-1)[src, None].double() * x.double().cpu()[src // top]).to(torch.bfloat16)
    assert torch.equal(a.cpu(), want_a)
    w = rnd((experts, inner, k), 2, 0.2).to(torch.bfloat16).to(DEV)
    out = torch.empty(rows * top, inner, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().moe_gemm_tcgen05(a, w, out, offsets, status, unary="relu2")
    assert status.item() == 0
    off = offsets.cpu().tolist()
    for e in range(experts):
        if off[e] == off[e + 1]:
            continue
        rows_e = a[off[e]:off[e + 1]].double().cpu()
        want = torch.relu(rows_e @ w[e].double().cpu().T) ** 2
        close(out[off[e]:off[e + 1]], want, "bfloat16", e)


# ------------------------------------------------------------------------------------------------ whole models

@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("reverax")
    return {name: tr.make_folder(tmp, raw, seed=i + 1) for i, (name, (raw, _)) in enumerate(tr.CONFIGS.items())}


_plain_memo = {}


def plain_logits(folder, raw, tokens):
    key = (folder, tuple(tokens))
    if key not in _plain_memo:
        _plain_memo[key] = plain.forward(raw, tr.weights(folder), tokens)
    return _plain_memo[key]


def clear_choices(folder, raw, tokens, least=0.03):
    """[T] bool: rows of which every routed layer chooses its experts by a margin that bfloat16 rounding cannot turn."""
    margins = []
    plain.forward(raw, tr.weights(folder), tokens, margins_out=margins)
    ok = torch.ones(len(tokens), dtype=torch.bool)
    for m in margins:
        ok &= m > least
    return ok


def bfloat16_rows_agree(got: dict, want: dict, clear: dict, bound, what):
    """A row whose experts are chosen by a clear margin, behind rows of its request that all are, lies within ``bound``: no
    other choice reaches it through keys, values or the state.  (A row where bfloat16 rounding turns a close call takes
    another expert, which changes it by far more than rounding does, and every later row of the request reads it through the
    window's keys and the state.)  Of all rows with clear choices of their own at most one in twenty lies beyond the bound,
    and the median of all rows stays small."""
    errs, clears = [], []
    for rid in got:
        err = tr.row_error(got[rid], want[rid])
        unclear = torch.nonzero(~clear[rid]).flatten()
        upto = int(unclear[0]) if unclear.numel() else err.numel()
        if upto:
            assert err[:upto].max().item() < bound, (what, rid, int(err[:upto].argmax()), err[:upto].max().item())
        errs.append(err)
        clears.append(clear[rid])
    err, ok = torch.cat(errs), torch.cat(clears)
    assert not torch.isnan(err).any() and ok.float().mean().item() > 0.3, what
    assert (err[ok] > bound).float().mean().item() <= 0.05, (what, (err[ok] > bound).float().mean().item())
    assert err.median().item() < 0.06, (what, err.median().item())


def requests_for(raw, lengths, seed):
    return {f"q{i}": p for i, p in enumerate(tiny.prompts(raw["vocab"], lengths, seed=seed))}


WAYS = {"whole": replay.whole, "tail": lambda r: replay.tail_one_by_one(r, 40), "portions": replay.portions, "mixed": replay.mixed}
LENGTHS = {"R1": [150, 1, 2, 61, 34, 97], "R2": [260, 70, 1, 129, 3], "R3": [300, 3, 66, 2, 131], "R4": [120, 8, 2, 57]}


@pytest.mark.parametrize("name", ["R1", "R2", "R3", "R4"])
def test_float32_replay_every_way_against_the_plain_implementation(folders, name):
    from rust_mlx_b200.engine import Engine
    raw, page = tr.CONFIGS[name]
    reqs = requests_for(raw, LENGTHS[name], seed=11)
    want = {rid: plain_logits(folders[name], raw, toks) for rid, toks in reqs.items()}
    first = None
    for way, cut in WAYS.items():
        steps = cut(reqs)
        # a cache just large enough and four slots: pages and slots are used again as requests end
        eng = Engine(folders[name], dtype="float32", max_tokens=replay.tokens_needed(steps, page), page_size=page, max_requests=4)
        got = replay.run_engine(eng, steps)
        eng.pools.table.check()
        assert eng.pools.table.live() == 0
        for rid in reqs:
            err = tr.row_error(got[rid], want[rid])
            assert err.max().item() < 2e-4, (name, way, rid, int(err.argmax()), err.max().item())
        if first is None:
            first = got
        else:       # the way of cutting changes nothing: every sum's order follows positions and sizes alone
            for rid in reqs:
                assert torch.equal(got[rid], first[rid]), (name, way, rid)


@pytest.mark.parametrize("name", ["R1", "R2", "R3", "R4"])
def test_bfloat16_replay_every_way(folders, name):
    from rust_mlx_b200.engine import Engine
    raw, page = tr.CONFIGS[name]
    reqs = requests_for(raw, LENGTHS[name], seed=12)
    want = {rid: plain_logits(folders[name], raw, toks) for rid, toks in reqs.items()}
    clear = {rid: clear_choices(folders[name], raw, toks) for rid, toks in reqs.items()}
    for way, cut in WAYS.items():
        steps = cut(reqs)
        eng = Engine(folders[name], dtype="bfloat16", max_tokens=replay.tokens_needed(steps, page), page_size=page, max_requests=4)
        got = replay.run_engine(eng, steps)
        eng.pools.table.check()
        bfloat16_rows_agree(got, want, clear, 0.15, (name, way))


def test_every_layer_against_the_plain_implementation(folders):
    """The stream after every layer, in 32-bit: a difference is found at the first layer that shows it."""
    from rust_mlx_b200.engine import Engine
    for name in ("R1", "R2", "R3", "R4"):
        raw, page = tr.CONFIGS[name]
        toks = tiny.prompts(raw["vocab"], [45], seed=5)[0]
        layers = []
        plain.forward(raw, tr.weights(folders[name]), toks, layers_out=layers)
        eng = Engine(folders[name], dtype="float32", max_tokens=128, page_size=page, max_requests=2)
        _, taken = eng.step_with_intermediates([("a", toks, [])], ["a"])
        assert len(eng.spec.schedule) == len(layers)
        for r in range(len(layers) - 1):
            got = taken[f"run{r + 1}.residual"].double().cpu()
            assert (got - layers[r]).abs().max().item() < 1e-4 * (1 + layers[r].abs().max().item()), (name, r)


def needle_model(tmp_path, kind, window=0):
    """One layer whose mixer decides: scores spread so widely that single keys carry a row's weight."""
    if kind == "talk":
        mixer = tr.talk(4, 2, 16, 16, tr.rot(1e4, 8), scale=0.3)
    else:
        mixer = tr.side(2, 1, 16, 16, tr.rot(1e4, 8), window, 0.0, 1, 8, 2, 1.0, 0.05, scale=0.3)
    raw = tr.model(90, 48, [tr.layer(mixer, None)])
    return raw, tr.make_folder(tmp_path, raw, seed=5, sharp=40.0, out_boost=30.0)


def test_far_keys_decide_and_are_found_in_prompts_and_in_decoding(tmp_path):
    from rust_mlx_b200.engine import Engine
    raw, folder = needle_model(tmp_path, "talk")
    toks = tiny.prompts(90, [520], seed=3)[0]
    want = plain.forward(raw, tr.weights(folder), toks)
    for cut in (replay.whole, lambda r: replay.tail_one_by_one(r, 60), replay.portions):
        steps = cut({"a": toks})
        eng = Engine(folder, dtype="float32", max_tokens=replay.tokens_needed(steps, 16), page_size=16, max_requests=2)
        got = replay.run_engine(eng, steps)["a"]
        assert tr.row_error(got, want).max().item() < 2e-4
    # the plain implementation itself, told to forget what is older than 300 positions, gives other logits
    see = plain.visible
    try:
        plain.visible = lambda t, window: see(t, 300)
        near = plain.forward(raw, tr.weights(folder), toks)
    finally:
        plain.visible = see
    assert tr.row_error(near[400:], want[400:]).max().item() > 0.05
    eng = Engine(folder, dtype="bfloat16", max_tokens=1024, page_size=16, max_requests=2)
    got = replay.run_engine(eng, replay.tail_one_by_one({"a": toks}, 60))["a"]
    err = tr.row_error(got, want)
    assert err.max().item() < 0.4 and err.median().item() < 0.08


@pytest.mark.parametrize("window, page", [(48, 16), (40, 64), (64, 64), (2, 16), (17, 16)])
def test_a_windows_edge_shows_in_the_logits_of_prompts_and_decoded_tokens(tmp_path, window, page):
    """With scores this sharp a window that is one position off (a key too many, a key too few) changes the logits by far
    more than the bound; rows are taken whole, decoded one by one past the window, and in small portions; pages that the
    window has passed are handed back on the way."""
    from rust_mlx_b200.engine import Engine
    raw, folder = needle_model(tmp_path, "side", window=window)
    toks = tiny.prompts(90, [3 * window + 70], seed=window)[0]
    want = plain.forward(raw, tr.weights(folder), toks)
    see = plain.visible
    for off in (-1, 1):
        try:
            plain.visible = lambda t, w: see(t, w + off if w else w)
            wrong = plain.forward(raw, tr.weights(folder), toks)
        finally:
            plain.visible = see
        assert tr.row_error(wrong, want).max().item() > 0.05
    for dtype, bound in (("float32", 2e-4), ("bfloat16", 0.3)):
        for cut in (replay.whole, lambda r: replay.tail_one_by_one(r, 2 * window + 60), replay.portions):
            steps = cut({"a": toks})
            eng = Engine(folder, dtype=dtype, max_tokens=replay.tokens_needed(steps, page), page_size=page, max_requests=2)
            got = replay.run_engine(eng, steps)["a"]
            assert tr.row_error(got, want).max().item() < bound, (dtype, window)


def test_the_state_carries_what_the_window_forgot(tmp_path):
    """A layer whose right mixer decides (decays near 1, the left scaled down): the first tokens of a sequence change rows
    hundreds of positions later, in prompts, in portions and in decoding; a state that was lost or reset would show."""
    from rust_mlx_b200.engine import Engine
    from safetensors.torch import load_file, save_file
    mixer = tr.side(2, 1, 16, 16, tr.rot(1e4, 8), 8, 0.0, 2, 16, 4, 0.05, 1.0, scale=0.3)
    raw = tr.model(90, 48, [tr.layer(mixer, None)])
    folder = tr.make_folder(tmp_path, raw, seed=8, out_boost=30.0)
    t = load_file(f"{folder}/model.safetensors")
    t["l0.mix.right.w0"] = torch.full_like(t["l0.mix.right.w0"], -6.0)       # a decay of exp(-exp(-6)) = 0.9975 a token
    save_file(t, f"{folder}/model.safetensors")
    w = tr.weights(folder)
    toks = tiny.prompts(90, [400], seed=4)[0]
    want = plain.forward(raw, w, toks)
    other = plain.forward(raw, w, [(toks[0] + 1) % 90, (toks[1] + 7) % 90] + toks[2:])
    assert tr.row_error(other[350:], want[350:]).min().item() > 1e-3          # the first two tokens still show at the end
    for cut in (replay.whole, lambda r: replay.tail_one_by_one(r, 120), replay.portions):
        steps = cut({"a": toks})
        eng = Engine(folder, dtype="float32", max_tokens=replay.tokens_needed(steps, 16), page_size=16, max_requests=2)
        assert tr.row_error(replay.run_engine(eng, steps)["a"], want).max().item() < 2e-4


def test_pages_and_slots_that_are_used_again_give_the_same_bits(folders):
    """Two slots and pages for one long request: every request takes over what the one before it left (keys and states of
    another request); the same request run again gives the same bits as in a fresh engine."""
    from rust_mlx_b200.engine import Engine
    raw, page = tr.CONFIGS["R1"]
    prompts = tiny.prompts(raw["vocab"], [70, 40, 70, 9], seed=9)
    fresh = []
    for p in prompts:
        eng = Engine(folders["R1"], dtype="float32", max_tokens=128, page_size=page, max_requests=2)
        half = len(p) // 2
        eng.step([("x", p[:half], [])])
        fresh.append(eng.step([("x", p[half:], list(range(len(p) - half)))], ["x"]).cpu())
    eng = Engine(folders["R1"], dtype="float32", max_tokens=128, page_size=page, max_requests=2)
    for turn in range(2):
        for i, p in enumerate(prompts):
            half = len(p) // 2
            eng.step([((turn, i), p[:half], [])])
            got = eng.step([((turn, i), p[half:], list(range(len(p) - half)))], [(turn, i)]).cpu()
            assert torch.equal(got, fresh[i]), (turn, i)
    eng.pools.table.check()


def test_a_request_in_a_batch_equals_the_request_alone(folders):
    """Unequal requests side by side (a long portion, single tokens, two tokens) against each alone, in both dtypes."""
    from rust_mlx_b200.engine import Engine
    for name in ("R1", "R3"):
        raw, page = tr.CONFIGS[name]
        prompts = tiny.prompts(raw["vocab"], [140, 33, 2, 71], seed=17)
        for dtype, bound in (("float32", 0.0), ("bfloat16", 0.08)):
            alone = []
            for p in prompts:
                eng = Engine(folders[name], dtype=dtype, max_tokens=256, page_size=page, max_requests=4)
                eng.step([("x", p[:-1], [])])
                alone.append(eng.step([("x", p[-1:], [0])], ["x"]).float().cpu())
            eng = Engine(folders[name], dtype=dtype, max_tokens=512, page_size=page, max_requests=4)
            eng.step([(0, prompts[0][:-1], []), (1, prompts[1][:-1], [])])
            got = eng.step([(0, prompts[0][-1:], [0]), (2, prompts[2], [1]), (1, prompts[1][-1:], [0]), (3, prompts[3][:-1], [])], [0, 1, 2]).float().cpu()
            last = eng.step([(3, prompts[3][-1:], [0])], [3]).float().cpu()
            for row, i in ((got[0], 0), (got[1], 2), (got[2], 1), (last[0], 3)):
                assert tr.row_error(row[None], alone[i]).item() <= bound, (name, dtype, i)


def test_long_decoding(folders):
    from rust_mlx_b200.engine import Engine
    raw, page = tr.CONFIGS["R1"]
    toks = tiny.prompts(raw["vocab"], [330], seed=21)[0]
    want = plain_logits(folders["R1"], raw, toks)
    eng = Engine(folders["R1"], dtype="float32", max_tokens=512, page_size=page, max_requests=2)
    got = replay.run_engine(eng, replay.tail_one_by_one({"a": toks}, 325))["a"]
    assert tr.row_error(got, want).max().item() < 2e-4


def greedy(raw, w, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(plain.forward(raw, w, ids)[-1].argmax()))
    return ids[len(prompt):]


def test_greedy_generation_through_the_scheduler(folders):
    from rust_mlx_b200.engine import Engine
    for name in ("R1", "R4"):
        raw, page = tr.CONFIGS[name]
        w = tr.weights(folders[name])
        prompts = tiny.prompts(raw["vocab"], [30, 3, 55, 9, 41], seed=31)
        want = [greedy(raw, w, p, 8) for p in prompts]
        # a cache too small for all five at once and three slots: requests wait, step back and are computed again
        eng = Engine(folders[name], dtype="float32", max_tokens=4 * page * 2 + 2 * page, page_size=page, max_requests=3)
        got = eng.generate(prompts, max_tokens=8, prefill_chunk=13, ignore_eos=True)
        assert got == want, name
        eng.pools.table.check()


def test_generation_in_graphs_equals_plain_launches(folders):
    from rust_mlx_b200.engine import Engine
    for name in ("R3", "R1"):
        raw, page = tr.CONFIGS[name]
        w = tr.weights(folders[name])
        prompts = tiny.prompts(raw["vocab"], [70, 9, 140, 33, 5], seed=41)
        exact = [Engine(folders[name], dtype="float32", max_tokens=4096, page_size=page, max_requests=8, cuda_graphs=g)
                 .generate(prompts, max_tokens=12, prefill_chunk=64, ignore_eos=True) for g in (True, False)]
        assert exact[0] == exact[1], name
        eng = Engine(folders[name], dtype="bfloat16", max_tokens=4096, page_size=page, max_requests=8)
        assert eng.graphs is not None
        got = eng.generate(prompts, max_tokens=12, prefill_chunk=64, ignore_eos=True)
        assert eng.graphs.replays > 0
        plain_steps = Engine(folders[name], dtype="bfloat16", max_tokens=4096, page_size=page, max_requests=8, cuda_graphs=False)
        assert plain_steps.generate(prompts, max_tokens=12, prefill_chunk=64, ignore_eos=True) == got
        for p, g in zip(prompts, got):
            ids = list(p)
            for t in g:
                logits = plain.forward(raw, w, ids)[-1]
                spread = (logits - logits.mean()).pow(2).mean().sqrt()
                assert logits[t] >= logits.max() - 0.2 * spread, (name, t, int(logits.argmax()))
                ids.append(t)


def test_trace_tool_and_command_line_run_this_design(folders, tmp_path):
    import json
    import os
    import subprocess
    import sys
    raw, page = tr.CONFIGS["R1"]
    reqs = requests_for(raw, [40, 1, 77, 20, 5], seed=51)
    steps = replay.mixed(reqs)
    got = replay.run_trace_tool(folders["R1"], "float32", steps, str(tmp_path / "out"), replay.tokens_needed(steps, 64), raw["vocab"])
    for rid, toks in reqs.items():
        assert tr.row_error(got[rid], plain_logits(folders["R1"], raw, toks)).max().item() < 2e-4
    prompt = tiny.prompts(raw["vocab"], [12], seed=2)[0]
    ids, report = str(tmp_path / "prompt.json"), str(tmp_path / "report.json")
    json.dump(prompt, open(ids, "w"))
    cmd = [sys.executable, os.path.join(replay.ROOT, "bin", "infer"), "--model", folders["R1"], "--prompt-ids", ids, "--max-tokens", "6", "--runs", "2",
           "--warmup-tokens", "2", "--prefill-chunk", "5", "--ignore-eos", "--dtype", "float32", "--page-size", "16", "--output", report]
    subprocess.run(cmd, check=True, timeout=300)
    want = greedy(raw, tr.weights(folders["R1"]), prompt, 6)
    assert [r["tokens"] for r in json.load(open(report))["runs"]] == [want, want]


def random_configuration(seed):
    """Sizes, head counts, the order and number of layers, windows, groups and every constant drawn from a seed."""
    r = random.Random(seed)
    layers = []
    for i in range(r.randint(2, 4)):
        if r.random() < 0.5:
            kv = r.choice([1, 2, 3])
            dim = r.choice([8, 12, 16, 24])
            mixer = tr.talk(kv * r.choice([1, 2, 3]), kv, dim, r.choice([6, 8, 16, 20]), tr.rot(r.choice([50.0, 1e4, 3e5]), r.choice([0, 4, dim])),
                            scale=r.choice([0.2, 0.5]))
        else:
            kv = r.choice([1, 2])
            dim = r.choice([8, 16, 32])
            mixer = tr.side(kv * r.choice([1, 2, 4]), kv, dim, r.choice([6, 8, 16, 32]), tr.rot(r.choice([50.0, 1e4, 3e5]), r.choice([0, 4, dim])),
                            r.choice([0, 1, 5, 16, 33]), r.choice([0.0, 4.0, 30.0]), r.choice([1, 2, 3]), r.choice([6, 8, 16, 20]), r.choice([1, 3, 8]),
                            r.choice([0.5, 1.0, 1.2]), r.choice([0.7, 1.0, 1.1]), scale=r.choice([0.2, 0.5]))
        kind = r.random()
        if kind < 0.25:
            mlp = None
        elif kind < 0.55:
            mlp = tr.dense(r.choice([20, 64]))
        else:
            e = r.choice([1, 3, 8])
            mlp = tr.moe(r.choice([12, 64]), e, r.randint(1, min(e, 3)))
        layers.append(tr.layer(mixer, mlp))
    if r.random() < 0.6:       # some layer again with caches of its own, somewhere later
        j = r.randrange(len(layers))
        layers.insert(r.randint(j + 1, len(layers)), {**layers[j], "weights_of": j})
        for i, layer in enumerate(layers):      # (indices of owners behind the inserted layer do not move: it is inserted after j)
            if "weights_of" in layer:
                layer["weights_of"] = j
    groups = r.choice([1, 2, 4])
    width = groups * r.choice([10, 16, 24])
    return tr.model(r.choice([61, 128, 200]), width, layers, eps=r.choice([1e-6, 1e-5, 1e-3]), groups=groups, logit_scale=r.choice([None, 0.5, 2.0]))


@pytest.mark.parametrize("seed", range(8))
def test_random_configurations_replayed_in_mixed_steps(tmp_path, seed):
    from rust_mlx_b200.engine import Engine
    raw = random_configuration(seed)
    folder = tr.make_folder(tmp_path, raw, seed=seed)
    page = [16, 32, 64][seed % 3]
    reqs = requests_for(raw, [90, 2, 41, 130, 7], seed=seed)
    want = {rid: plain.forward(raw, tr.weights(folder), toks) for rid, toks in reqs.items()}
    for cut in (replay.mixed, replay.portions):
        steps = cut(reqs)
        eng = Engine(folder, dtype="float32", max_tokens=replay.tokens_needed(steps, page), page_size=page, max_requests=4)
        got = replay.run_engine(eng, steps)
        for rid in reqs:
            assert tr.row_error(got[rid], want[rid]).max().item() < 2e-4, (seed, rid)
    steps = replay.mixed(reqs)
    eng = Engine(folder, dtype="bfloat16", max_tokens=replay.tokens_needed(steps, page), page_size=page, max_requests=4)
    got = replay.run_engine(eng, steps)
    bfloat16_rows_agree(got, want, {rid: clear_choices(folder, raw, toks) for rid, toks in reqs.items()}, 0.3, seed)
