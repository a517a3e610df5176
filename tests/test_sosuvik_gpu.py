"""Sosuvik on the GPU against its plain implementation (tests/plain_sosuvik.py): every mechanism alone, then whole models
replayed in every way of cutting, in both dtypes, through the engine's step function, scheduler and command line."""
import math
import random

import pytest
import torch

import plain_sosuvik as plain
import replay
import tiny
import tiny_sosuvik as ts
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


def bind(part, seed=0, dtype=torch.float32, scale=None):
    """Random tensors for ``part`` (``scale``: name ending -> factor), bound; returns them in float64 on the host."""
    from rust_mlx_b200.weights.random_init import random_tensors
    tensors = random_tensors(part.all_param_specs(), seed, dtype, DEV)
    for ending, factor in (scale or {}).items():
        for k in tensors:
            if k.endswith(ending):
                tensors[k] = (tensors[k].float() * factor).to(tensors[k].dtype)
    host = {k: v.detach().cpu().to(F) for k, v in tensors.items()}
    part.bind_all(tensors, context(dtype))
    return host


# ------------------------------------------------------------------------------------------------ kernels alone

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows, width", [(1, 64), (37, 90), (300, 336), (5, 4096), (2, 6)])
def test_two_norms_of_one_sum(dtype, rows, width):
    """h + mult * (a + ratio * b) is stored once, and normed twice with two weights."""
    dt = DT[dtype]
    h = rnd((rows, width), 1, 3.0)
    a, b = rnd((rows, width), 2).to(dt), rnd((rows, width), 3).to(dt)
    w1, w2 = 1 + rnd((width,), 4, 0.3), rnd((width,), 5)
    hd = h.to(DEV)
    x1 = torch.full((rows, width), float("nan"), dtype=dt, device=DEV)
    x2 = torch.full_like(x1, float("nan"))
    ops().add_rmsnorm(hd, a.to(DEV), w1.to(DEV), 1e-5, x1, delta2=b.to(DEV), mult=0.5, mult2=2.0, weight2=w2.to(DEV), x2_out=x2)
    total = h.double() + 0.5 * (a.double() + 2.0 * b.double())
    close(hd, total, "float32")
    stored = hd.double().cpu()
    close(x1, plain.rms_norm(stored, w1.double(), 1e-5), dtype)
    close(x2, plain.rms_norm(stored, w2.double(), 1e-5), dtype)
    # nothing to add: the stream stays as it is, bit for bit
    before = hd.clone()
    ops().add_rmsnorm(hd, None, w1.to(DEV), 1e-5, x1, weight2=w2.to(DEV), x2_out=x2)
    assert torch.equal(hd, before)
    close(x2, plain.rms_norm(stored, w2.double(), 1e-5), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows, width", [(1, 64), (41, 90), (7, 336), (3, 2)])
def test_stream_beside_the_embedding_rows(dtype, rows, width):
    dt = DT[dtype]
    h = rnd((rows, width), 1, 3.0)
    a, b, x0 = rnd((rows, width), 2).to(dt), rnd((rows, width), 3).to(dt), rnd((rows, width), 4).to(dt)
    for write in (False, True):
        hd = h.to(DEV)
        out = torch.full((rows, 2 * width), float("nan"), dtype=dt, device=DEV)
        ops().stream_concat(hd, a.to(DEV), x0.to(DEV), out, delta2=b.to(DEV), mult=1.0, mult2=1.0, write_h=write)
        total = h.double() + a.double() + b.double()
        close(out[:, :width], total, dtype)
        assert torch.equal(out[:, width:].cpu(), x0)
        if write:
            close(hd, total, "float32")
        else:
            assert torch.equal(hd.cpu(), h)
    hd = h.to(DEV)
    ops().stream_concat(hd, None, x0.to(DEV), out)          # the first layer of a model: nothing is pending
    close(out[:, :width], h.double(), dtype)


def chunked_rows(q, k, v, qpos, chunk, cap, scale, sink):
    """q [T, nq, d] at positions qpos over keys 0..S-1 -> [T, nq, dv]: the plain mechanisms put together."""
    T, nq, _ = q.shape
    group = nq // k.shape[1]
    kpos = torch.arange(k.shape[0])
    ok = kpos[None, :] <= qpos[:, None]
    if chunk:
        ok &= (kpos[None, :] // chunk) == (qpos[:, None] // chunk)
    out = torch.empty(T, nq, v.shape[2], dtype=F)
    for h in range(nq):
        s = (q[:, h].double() @ k[:, h // group].double().t()) * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(~ok, -math.inf)
        p = plain.softmax_with_sink(s) if sink else torch.softmax(s, -1)
        out[:, h] = p @ v[:, h // group].double()
    return out


def run_attention(kernel, q, k_pool, v_pool, batch, table, page, nq, nkv, hd, scale, chunk, cap, sink, variant=None):
    from rust_mlx_b200.engine.workspace import Workspace
    out = torch.full_like(q, float("nan"))
    sinks = torch.zeros(nq, dtype=torch.float32, device=DEV) if sink else None
    ws = Workspace(DEV)
    if kernel == "plain":
        ops().attention_plain(q, k_pool, v_pool, batch.positions, batch.seq_index, table, page, out, nq, nkv, hd, 0, scale, batch.status,
                              sinks, chunk, cap)
    elif kernel == "flash":
        ops().attention_flash(q, k_pool, v_pool, batch, table, page, out, nq, nkv, hd, 0, scale, ws, n_splits=variant, sinks=sinks,
                              chunk=chunk, softcap=cap)
    elif kernel == "tcgen05":
        per_block, runs = variant or (None, None)
        ops().attention_tcgen05(q, k_pool, v_pool, batch, table, page, out, nq, nkv, hd, 0, scale, per_block=per_block, n_splits=runs,
                                workspace=ws, sinks=sinks, chunk=chunk, softcap=cap)
    else:       # the engine's own choice of kernels for the step
        ops().default.attention(q, k_pool, v_pool, batch, table, page, out, nq, nkv, hd, 0, scale, ws, sinks=sinks, chunk=chunk, softcap=cap)
    assert batch.status.item() == 0
    return out


VARIANTS = {"plain": [None], "flash": [None, 1, 3], "tcgen05": [None, (2, 1), (1, 3)], "engine": [None]}


@pytest.mark.parametrize("dtype, nq, nkv, hd, page, kernel", [
    ("float32", 6, 3, 24, 16, "plain"), ("bfloat16", 4, 1, 48, 8, "plain"), ("float32", 2, 2, 64, 64, "plain"),
    ("bfloat16", 6, 2, 64, 16, "flash"), ("bfloat16", 4, 4, 32, 16, "flash"), ("bfloat16", 8, 2, 128, 64, "flash"),
    ("bfloat16", 8, 2, 64, 64, "tcgen05"), ("bfloat16", 4, 4, 128, 64, "tcgen05"), ("bfloat16", 8, 4, 64, 64, "engine"),
    ("bfloat16", 6, 2, 128, 32, "engine")])
@pytest.mark.parametrize("chunk, cap, sink", [(50, 4.0, True), (64, 0.0, True), (176, 7.5, False), (7, 2.0, True), (0, 3.0, True), (1000, 0.0, False)])
def test_chunked_capped_attention_with_a_sink_in_every_kernel(dtype, nq, nkv, hd, page, kernel, chunk, cap, sink):
    """Portions that start inside a chunk and run over several, decoded tokens at a chunk's first and last place, long
    sequences whose chunk is a small part of them; scores large enough that the cap bends them; NaN in every place of
    the pool that holds no key."""
    dt = DT[dtype]
    lengths, new = [700, 1, 33, 130, 301, 64, 1500, 400, 201], [260, 1, 33, 1, 1, 64, 1, 1, 2]
    k_pool, v_pool, table, ks, vs = paged_setup(lengths, nkv, hd, page, dt, seed=hd + nq)
    qs = [(rnd((c, nq, hd), 70 + i) * 1.5).to(dt) for i, c in enumerate(new)]
    q = torch.cat(qs).to(DEV).reshape(-1, nq * hd)
    scale = 1.3 * hd ** -0.5
    for variant in VARIANTS[kernel]:
        batch = _Batch(lengths, new, torch.zeros(1, dtype=torch.int32, device=DEV))
        out = run_attention(kernel, q, k_pool, v_pool, batch, table, page, nq, nkv, hd, scale, chunk, cap, sink, variant)
        at = 0
        for s, (n, c) in enumerate(zip(lengths, new)):
            want = chunked_rows(qs[s], ks[s], vs[s], torch.arange(n - c, n), chunk, cap, scale, sink)
            got = out[at:at + c].double().cpu().reshape(c, nq, hd)
            assert not torch.isnan(got).any(), (variant, s, n, c)
            tol = 1.5e-2 if dtype == "bfloat16" else 2e-5
            assert ((got - want).abs() <= tol * (1 + want.abs())).all(), (variant, s, n, c, (got - want).abs().max().item())
            at += c


@pytest.mark.parametrize("kernel, dtype, hd, page", [("plain", "float32", 16, 4), ("plain", "float32", 32, 16), ("flash", "bfloat16", 64, 16),
                                                     ("flash", "bfloat16", 32, 64), ("tcgen05", "bfloat16", 64, 64), ("tcgen05", "bfloat16", 128, 16),
                                                     ("engine", "bfloat16", 64, 64)])
@pytest.mark.parametrize("chunk", [48, 64, 50])
def test_a_chunks_first_key_is_seen_and_the_key_before_it_is_not(kernel, dtype, hd, page, chunk):
    """One key carries a score far above all others: at the first place of the query's chunk it takes nearly all the weight
    (what is left is the sink's and the others'), one place earlier it must not show at all.  The query is decoded alone,
    the last row of a long portion, and a row in the middle of a portion that began in the chunk before."""
    dt = DT[dtype]
    nq, nkv = 4, 2
    n = 5 * chunk + 9                      # the last query sits nine places into the sixth chunk
    first = 5 * chunk
    k_pool, v_pool, table, ks, vs = paged_setup([n], nkv, hd, page, dt, seed=chunk + hd)
    for new, row in ((1, 0), (chunk + 20, chunk + 19), (chunk + 30, chunk + 19)):
        length = n if new != chunk + 30 else n + 11             # (the third: eleven more rows follow the query's)
        kp, vp, tb, kk, vv = (k_pool, v_pool, table, ks, vs) if length == n else paged_setup([length], nkv, hd, page, dt, seed=chunk + hd)
        qpos = length - new + row
        assert qpos // chunk == 5
        for target, seen in ((first, True), (first - 1, False)):
            k2 = kp.clone()
            k2[int(tb[0, target // page]), :, target % page, :] = 0
            k2[int(tb[0, target // page]), :, target % page, 0] = 24.0
            q = (rnd((new, nq, hd), 9) * 0.05).to(dt)
            q[row, :, 0] = 24.0
            batch = _Batch([length], [new], torch.zeros(1, dtype=torch.int32, device=DEV))
            out = run_attention(kernel, q.reshape(new, nq * hd).to(DEV), k2, vp, batch, tb, page, nq, nkv, hd, 0.05, chunk, 0.0, True)
            got = out[row].double().cpu().view(nq, hd)
            hit = vv[0][target].double().repeat_interleave(nq // nkv, 0)
            near = (got - hit).abs().max().item() < 0.05 * (1 + hit.abs().max().item())
            assert near == seen, (new, row, target, seen)
            kf = kk[0].clone()
            kf[target] = 0
            kf[target, :, 0] = 24.0
            want = chunked_rows(q[row:row + 1], kf, vv[0], torch.tensor([qpos]), chunk, 0.0, 0.05, True)[0]
            assert ((got - want).abs() <= (2e-2 if dtype == "bfloat16" else 2e-5) * (1 + want.abs())).all()


def test_the_cap_bounds_a_score_and_the_sink_takes_its_share():
    """One key, one query: the weight of the key is exp(c) / (1 + exp(c)) with c = cap * tanh(s / cap)."""
    nq, nkv, hd, page = 2, 1, 16, 8
    k_pool, v_pool, table, ks, vs = paged_setup([1], nkv, hd, page, torch.float32, seed=1)
    for s_raw, cap in ((0.3, 0.0), (5.0, 2.0), (-6.0, 1.5), (100.0, 3.0), (0.4, 50.0)):
        q = torch.zeros(1, nq, hd)
        q[0, :, 0] = s_raw
        k_pool[int(table[0, 0]), :, 0, :] = 0
        k_pool[int(table[0, 0]), :, 0, 0] = 1.0
        batch = _Batch([1], [1], torch.zeros(1, dtype=torch.int32, device=DEV))
        out = run_attention("plain", q.reshape(1, -1).to(DEV), k_pool, v_pool, batch, table, page, nq, nkv, hd, 1.0, 0, cap, True)
        c = cap * math.tanh(s_raw / cap) if cap else s_raw
        share = math.exp(c) / (1 + math.exp(c))
        close(out.view(nq, hd), vs[0][0].double().expand(nq, hd) * share, "float32", (s_raw, cap))


@pytest.mark.parametrize("nq, nkv, dq, dv, hd, rot, page, pad", [
    (4, 2, 64, 64, 64, 32, 16, 0), (6, 3, 48, 24, 64, 16, 8, 8), (2, 2, 128, 128, 128, 128, 64, 0), (8, 1, 32, 40, 48, 0, 16, 16),
    (3, 1, 24, 24, 24, 8, 8, 0), (2, 2, 20, 12, 20, 20, 4, 3)])
@pytest.mark.parametrize("write", [True, False])
def test_unnormed_projection_split_rotated_and_written(nq, nkv, dq, dv, hd, rot, page, pad, write):
    """Rows [q | k | v] of a wider buffer, no norms: q heads (rotated over their first ``rot`` numbers, halves paired, padded
    with zeros to ``hd``) to their rows, k and v heads into the pages of tokens at scattered positions; every other place of
    the pools keeps its NaN.  Sizes in eights take the kernel of eight numbers a thread, the others the general one."""
    dt = torch.bfloat16
    lengths, new = [37, 5, 130], [9, 5, 1]
    starts = [n - c for n, c in zip(lengths, new)]
    n = sum(new)
    cols = (nq + nkv) * dq + nkv * dv
    buf = (rnd((n, cols + pad), 5) * 3).to(dt).to(DEV)
    qkv = buf[:, :cols]
    positions = torch.tensor([s + i for s, c in zip(starts, new) for i in range(c)], dtype=torch.int32, device=DEV)
    seq_index = torch.tensor([j for j, c in enumerate(new) for _ in range(c)], dtype=torch.int32, device=DEV)
    pages = [-(-L // page) for L in lengths]
    order = torch.randperm(sum(pages), generator=torch.Generator().manual_seed(nq)).tolist()
    table = torch.full((len(lengths), max(pages)), -1, dtype=torch.int32)
    for j, c in enumerate(pages):
        table[j, :c] = torch.tensor([order.pop() for _ in range(c)])
    table = table.to(DEV)
    k_pool = torch.full((sum(pages), nkv, page, hd), float("nan"), dtype=dt, device=DEV)
    v_pool = torch.full_like(k_pool, float("nan"))
    q_out = torch.full((n, nq * hd), float("nan"), dtype=dt, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    inv_freq = (1000.0 ** (-torch.arange(rot // 2, dtype=F) * 2 / max(rot, 1))).float().to(DEV) if rot else None
    cos_sin = None
    if rot:
        cos_sin = torch.empty(n, rot, dtype=torch.float32, device=DEV)
        ops().rope_table(positions, inv_freq, rot, cos_sin, 1.25)
    ops().qk_whole_norm_rope_cache(qkv, None, None, 0.0, inv_freq, rot, positions, seq_index, table, page, k_pool, v_pool, q_out,
                                   nq, nkv, dq, dv, hd, write, status, cos_sin)
    assert status.item() == 0
    x = qkv.double().cpu()
    heads = x[:, :(nq + nkv) * dq].reshape(n, nq + nkv, dq).clone()
    if rot:
        ang = positions.double().cpu()[:, None] * inv_freq.double().cpu()[None, :]
        cs, sn = (1.25 * torch.cos(ang))[:, None, :], (1.25 * torch.sin(ang))[:, None, :]
        a, b = heads[..., :rot // 2].clone(), heads[..., rot // 2:rot].clone()
        heads[..., :rot // 2], heads[..., rot // 2:rot] = a * cs - b * sn, b * cs + a * sn
    want_q = torch.zeros(n, nq, hd, dtype=F)
    want_q[..., :dq] = heads[:, :nq]
    close(q_out.reshape(n, nq, hd), want_q, "bfloat16")
    assert (q_out.reshape(n, nq, hd)[..., dq:] == 0).all()
    seen = torch.zeros(k_pool.shape[0], page, dtype=torch.bool)
    if write:
        for t in range(n):
            pos, pg = int(positions[t]), int(table[int(seq_index[t]), int(positions[t]) // page])
            seen[pg, pos % page] = True
            want_k = torch.zeros(nkv, hd, dtype=F)
            want_k[:, :dq] = heads[t, nq:]
            close(k_pool[pg, :, pos % page], want_k, "bfloat16")
            want_v = torch.zeros(nkv, hd, dtype=F)
            want_v[:, :dv] = x[t, (nq + nkv) * dq:].reshape(nkv, dv)
            assert torch.equal(v_pool[pg, :, pos % page].double().cpu(), want_v)
    untouched = ~seen[:, None, :, None].expand(-1, nkv, -1, hd)
    assert torch.isnan(k_pool.cpu()[untouched]).all() and torch.isnan(v_pool.cpu()[untouched]).all()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, dim, r, rot, row, page, neighbours", [(2, 16, 24, 8, 32, 16, True), (5, 6, 20, 6, 32, 4, True), (8, 32, 64, 64, 128, 64, True),
                                                                      (3, 8, 10, 4, 16, 8, False), (1, 4, 80, 48, 128, 16, True), (2, 14, 18, 2, 32, 8, True)])
def test_latent_and_rotated_key_part_into_a_page_row(dtype, heads, dim, r, rot, row, page, neighbours):
    """A page row becomes [norm(latent) | rotate(key part) | zeros]; a query row's rotated part lands behind the place that
    the latent's part takes, zeros behind it; what lies before is left alone."""
    dt = DT[dtype]
    lengths, new = [37, 5, 1, 70], [9, 5, 1, 2]
    n = sum(new)
    batch = _Batch(lengths, new, torch.zeros(1, dtype=torch.int32, device=DEV))
    qh = dim + rot
    wide = rnd((n, heads * qh + r + rot + 3), 7).to(dt)               # [queries | latent | key part | something else]
    w = 1 + rnd((r,), 8, 0.3)
    rotation = {"base": 300.0, "dims": rot}
    f, _ = plain.frequencies(rotation)
    pos = batch.positions.cpu()
    a = pos.double()[:, None] * f[None, :]
    cos_sin = torch.cat([torch.cos(a), torch.sin(a)], dim=1).float().to(DEV)
    n_pages = sum(-(-x // page) for x in lengths)
    pool = torch.full((n_pages, 1, page, row), float("nan"), dtype=dt, device=DEV)
    table, at = torch.full((len(lengths), max(-(-x // page) for x in lengths)), -1, dtype=torch.int32), 0
    for s, x in enumerate(lengths):
        for i in range(-(-x // page)):
            table[s, i] = n_pages - 1 - at
            at += 1
    wd = wide.to(DEV)
    q = wd[:, :heads * qh].unflatten(1, (heads, qh))
    q_out = torch.full((n, heads * row), 7.0, dtype=dt, device=DEV)
    ops().latent_rope(wd[:, heads * qh:heads * qh + r + rot], r, rot, neighbours, w.to(DEV), 1e-5, q, dim, heads, q_out, row, cos_sin, pool,
                      batch.positions, batch.seq_index, table.to(DEV), page, batch.status)
    assert batch.status.item() == 0
    x = wide.double()
    c = plain.rms_norm(x[:, heads * qh:heads * qh + r], w.double(), 1e-5)
    kr = plain.rotate(x[:, heads * qh + r:heads * qh + r + rot], pos, rotation, neighbours)
    qr = plain.rotate(x[:, :heads * qh].view(n, heads, qh)[:, :, dim:].transpose(0, 1), pos, rotation, neighbours).transpose(0, 1)
    got_q = q_out.double().cpu().view(n, heads, row)
    assert (got_q[:, :, :r] == 7.0).all()
    close(got_q[:, :, r:r + rot], qr, dtype)
    assert (got_q[:, :, r + rot:] == 0).all()
    for t in range(n):
        s, p = int(batch.seq_index[t]), int(pos[t])
        got = pool[int(table[s, p // page]), 0, p % page].double().cpu()
        close(got[:r], c[t], dtype)
        close(got[r:r + rot], kr[t], dtype)
        assert (got[r + rot:] == 0).all()
    assert torch.isnan(pool.float()).sum().item() == (n_pages * page - n) * row          # nothing else was written


ROUTERS = [  # experts, top, groups, keep, scale
    (8, 2, 4, 2, 2.5), (6, 3, 3, 2, 1.0), (9, 3, 3, 1, 0.5), (4, 2, 4, 2, 1.3), (12, 4, 1, 1, 1.0), (5, 5, 1, 1, 2.0), (16, 6, 4, 3, 1.0),
    (64, 8, 8, 4, 2.5), (8, 8, 2, 2, 1.0), (2, 1, 2, 1, 1.0), (40, 7, 5, 2, 0.7)]


@pytest.mark.parametrize("experts, top, groups, keep, scale", ROUTERS)
@pytest.mark.parametrize("corrected", ["none", "small", "negative"])
def test_router_chooses_by_corrected_scores_among_the_best_groups(experts, top, groups, keep, scale, corrected):
    """Against the plain choice.  'negative': every corrected score is below zero, so an expert of a group that is out,
    counted as 0, would win; 'small': corrections of the size of the scores' differences."""
    rows, width = 257, 48
    for dtype in ("float32", "bfloat16"):
        x = rnd((rows, width), experts).to(DT[dtype])
        wr = rnd((experts, width), top + 100, 0.4)
        correction = {"none": None, "small": rnd((experts,), 5, 0.3), "negative": rnd((experts,), 6, 0.3) - 3.0}[corrected]
        ids = torch.empty(rows, top, dtype=torch.int32, device=DEV)
        wts = torch.empty(rows, top, dtype=torch.float32, device=DEV)
        ops().moe_route(x.to(DEV), wr.to(DEV), top, ids, wts, scoring="sigmoid", correction=correction.to(DEV) if correction is not None else None,
                        groups=groups, keep=keep, route_scale=scale)
        z = x.double() @ wr.double().T
        router = {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}
        want_ids, want_w = plain.choose_experts(z, correction.double() if correction is not None else torch.zeros(experts, dtype=F), router)
        # (rows whose choice hangs on a difference that float rounding of the logits can turn are left out)
        c = torch.sigmoid(z) + (correction.double() if correction is not None else 0.0)
        gaps = (c.unsqueeze(1) - c.unsqueeze(2)).abs() + torch.eye(experts, dtype=F) * 9
        safe = gaps.flatten(1).min(-1).values > 1e-5
        if groups > 1:
            per = experts // groups
            worth = c.view(rows, groups, per).topk(min(2, per), dim=-1).values.sum(-1)
            wg = (worth.unsqueeze(1) - worth.unsqueeze(2)).abs() + torch.eye(groups, dtype=F) * 9
            safe &= wg.flatten(1).min(-1).values > 1e-5
        assert safe.sum().item() > rows * 0.9
        got = ids.long().cpu()
        assert torch.equal(got[safe], want_ids[safe]), (dtype, (got != want_ids).any(-1).nonzero().flatten()[:5])
        assert (wts.double().cpu()[safe] - want_w[safe]).abs().max().item() < 1e-5
        assert (wts.sum(-1).cpu() - scale).abs().max().item() < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n, inner, block", [(1, 88, 0), (37, 128, 64), (300, 40, 0), (5, 192, 64), (9, 7, 0)])
@pytest.mark.parametrize("limit, alpha", [(1.0, 1.702), (0.3, 1.702), (7.0, 1.0)])
def test_clamped_swish_times_up_plus_one(dtype, n, inner, block, limit, alpha):
    dt = DT[dtype]
    g, u = rnd((n, inner), 1, 2.0).to(dt), rnd((n, inner), 2, 2.0).to(dt)
    if block:
        rows = torch.stack([g.view(n, inner // block, block), u.view(n, inner // block, block)], dim=2).reshape(n, 2 * inner)
    else:
        rows = torch.cat([g, u], dim=1)
    out = torch.full((n, inner), float("nan"), dtype=dt, device=DEV)
    ops().swiglu(rows.to(DEV), out, block, "swish_clamp", (limit, alpha))
    gc, uc = g.double().clamp(max=limit), u.double().clamp(-limit, limit)
    close(out, gc * torch.sigmoid(alpha * gc) * (uc + 1.0), dtype)
    with pytest.raises(Exception):
        ops().swiglu(rows.to(DEV), out, block, "swish_clamp", ())


@pytest.mark.parametrize("rows, top, experts, inner, k", [(3, 2, 8, 128, 64), (64, 4, 6, 64, 200), (700, 2, 3, 192, 96), (2048, 3, 5, 256, 384)])
def test_experts_products_form_the_clamped_swish_in_their_epilogue(rows, top, experts, inner, k):
    """The tensor-core product over experts' runs with the activation in its epilogue, against the plain product and the
    pointwise kernel."""
    torch.manual_seed(rows)
    x = torch.randn(rows * top, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(experts, 2 * inner, k, device=DEV) * 0.2).to(torch.bfloat16)
    counts = torch.multinomial(torch.ones(experts), rows * top, replacement=True).bincount(minlength=experts)
    offsets = torch.tensor([0] + counts.cumsum(0).tolist(), dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    act = torch.full((rows * top, inner), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops().moe_gemm_tcgen05(x, w, act, offsets, status, gated=True, activation="swish_clamp", args=(0.8, 1.702))
    assert status.item() == 0
    owner = torch.repeat_interleave(torch.arange(experts), counts).to(DEV)
    gu = torch.einsum("pk,pnk->pn", x.double(), w[owner].double()).view(rows * top, inner // 64, 2, 64)
    g, u = gu[:, :, 0].reshape(rows * top, inner).clamp(max=0.8), gu[:, :, 1].reshape(rows * top, inner).clamp(-0.8, 0.8)
    want = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    assert ((act.double() - want).abs() <= 2e-2 * (1 + want.abs())).all()


# ------------------------------------------------------------------------------------------------ parts alone

def part_steps(mixer, x, cuts, page, dtype=torch.float32):
    """A mixer alone with a cache of its own, fed ``x`` in portions of the sizes ``cuts``."""
    from rust_mlx_b200.cache import CachePools
    from rust_mlx_b200.engine.batch import SequenceInput, build_batch
    pools = CachePools({0: mixer.cache_spec()}, max_tokens=-(-x.shape[0] // page) * page + page, page_size=page, max_requests=2, dtype=dtype,
                       device=DEV)
    for grp in pools.paged_groups:
        grp.k_pool.fill_(float("nan"))
        if grp.v_pool is not None:
            grp.v_pool.fill_(float("nan"))
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    pools.open(3)
    outs, at = [], 0
    for c in cuts:
        pools.table.reserve(3, at + c)
        batch = build_batch([SequenceInput(3, at, [0] * c, [])], pools, DEV, status, 10)
        outs.append(mixer.forward(x[at:at + c].contiguous(), batch, pools.view(0, batch, False)).clone())
        at += c
        pools.table.commit(3, at)
    assert status.item() == 0 and at == x.shape[0]
    return torch.cat(outs)


CUTS = (11, 1, 2, 1, 1, 7, 1, 1, 2, 19, 1, 3)


@pytest.mark.parametrize("heads, kv_heads, dim, vdim, dims, scaling, cap, chunk, page", [
    (4, 2, 16, 24, 8, (4.0, 64, 8.0, 2.0), 5.0, 12, 4), (3, 3, 8, 8, 8, None, 0.0, 0, 8), (6, 2, 16, 8, 4, None, 3.0, 5, 16),
    (2, 1, 12, 20, 12, (2.0, 16, 4.0, 1.0), 0.0, 16, 16), (1, 1, 16, 8, 8, None, 0.0, 0, 8)])
def test_attention_part_over_steps(heads, kv_heads, dim, vdim, dims, scaling, cap, chunk, page):
    from rust_mlx_b200.config.sosuvik import RotationConfig
    from rust_mlx_b200.parts.attention import GatedAttentionMixer
    from rust_mlx_b200.parts.position import RotaryEmbedding
    width = 40
    rot = ts.rot(777.0, dims, scaling)
    position = RotaryEmbedding(dim, 777.0, rotary_dim=dims, scaling=RotationConfig(777.0, dims, scaling).scaling_dict(), factor_on="rotated")
    mixer = GatedAttentionMixer("m", width, heads, kv_heads, dim, vdim, position, 0.3, sink=True, softcap=cap, chunk=chunk)
    w = bind(mixer, seed=heads, scale={".q": 25.0, ".k": 25.0, ".v": 20.0})
    x = rnd((sum(CUTS), width), 3).to(DEV)
    got = part_steps(mixer, x, CUTS, page)
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rot, "scale": 0.3}
    if cap:
        m["softcap"] = cap
    if chunk:
        m["mask"] = {"size": chunk}
    want = plain.chunked_attention(x.double().cpu(), w, "m", m)
    assert tiny.max_abs(got.cpu(), want) < 3e-5 * (1 + want.abs().max().item())


@pytest.mark.parametrize("heads, dim, rot_dim, vdim, kv_rank, page", [(2, 16, 8, 12, 24, 4), (5, 6, 6, 10, 20, 16), (3, 8, 16, 16, 40, 8),
                                                                      (20, 4, 4, 4, 8, 8)])
def test_latent_part_with_a_rotated_key_part_over_steps(heads, dim, rot_dim, vdim, kv_rank, page):
    """(Twenty heads: more than one attention launch takes.)"""
    from rust_mlx_b200.parts.latent_attention import LatentAttentionMixer
    from rust_mlx_b200.parts.position import RotaryEmbedding
    width = 40
    position = RotaryEmbedding(rot_dim, 500.0, rotary_dim=rot_dim, factor_on="rotated", interleaved=True)
    mixer = LatentAttentionMixer("m", width, heads, dim, vdim, 0, kv_rank, 1e-5, scale=0.25, gated=False, rot_dim=rot_dim, position=position)
    w = bind(mixer, seed=dim, scale={".q": 30.0, ".uk": 12.0, ".dkv": 30.0, ".uv": 10.0})
    x = rnd((sum(CUTS), width), 4).to(DEV)
    got = part_steps(mixer, x, CUTS, page)
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "rot": ts.rot(500.0, rot_dim), "scale": 0.25}
    want = plain.rotated_latent_attention(x.double().cpu(), w, "m", m, 1e-5)
    assert tiny.max_abs(got.cpu(), want) < 3e-5 * (1 + want.abs().max().item())
    # the rotated part matters: without it the plain result is another
    flat = plain.rotated_latent_attention(x.double().cpu(), {**w, "m.dkv": torch.cat([w["m.dkv"][:kv_rank], torch.zeros(rot_dim, width, dtype=F)])},
                                          "m", m, 1e-5)
    assert tiny.max_abs(flat, want) > 1e-2 * want.abs().max().item()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts, top, groups, keep, inner, rows", [(6, 2, 3, 2, 40, 37), (8, 3, 4, 2, 72, 300), (4, 4, 1, 1, 64, 5), (5, 1, 5, 1, 128, 64),
                                                                     (8, 2, 2, 1, 192, 700)])
def test_routed_part_with_groups_and_clamped_experts(dtype, experts, top, groups, keep, inner, rows):
    from rust_mlx_b200.parts.routed import RoutedFeedForward
    width = 64
    part = RoutedFeedForward("f", width, inner, experts, top, activation="swish_clamp", activation_args=(0.5, 1.702), scoring="sigmoid",
                             correction_name="correction", groups=groups, keep_groups=keep, route_scale=1.5)
    w = bind(part, seed=experts, dtype=DT[dtype], scale={".router": 30.0, ".correction": 10.0, ".gate": 20.0, ".up": 20.0, ".down": 10.0})
    x = rnd((rows, width), 7).to(DT[dtype])
    status = torch.zeros(1, dtype=torch.int32, device=DEV)

    class B:
        pass
    b = B()
    b.status = status
    got = part.forward(x.to(DEV), b).double().cpu()
    assert status.item() == 0
    mlp = {"expert": {"ff": inner, "limit": 0.5}, "router": {"experts": experts, "top": top, "scale": 1.5, "groups": {"count": groups, "keep": keep}}}
    want = plain.grouped_experts(x.double(), w, "f", mlp)
    err = (got - want).abs().max(-1).values / (1 + want.abs().max(-1).values)
    # (a row whose choice hangs on a rounding chooses another expert and differs much: such rows are few)
    bound = 2e-5 if dtype == "float32" else 3e-2
    assert (err < bound).float().mean().item() > 0.97, err.max().item()
    assert err.median().item() < bound


def test_loop_entry_mixes_the_embedding_rows_back_in():
    """x <- W_in [x; x0] + step[t], with what the layer before left still to be added to x: every pass has its own step
    vector and all share one product."""
    from rust_mlx_b200.parts.base import ScaledSum
    from rust_mlx_b200.parts.loop import LoopEntry
    width, times, rows = 40, 3, 23
    first = LoopEntry("lp.in", "lp.step", width, times, 0)
    others = [LoopEntry("lp.in", "lp.step", width, times, t, owner=first) for t in range(1, times)]
    w = bind(first, seed=3, scale={"lp.in": 20.0, "lp.step": 30.0})
    ctx = context()
    for o in others:
        assert o.param_specs() == []
        o.bind_all({}, ctx)
    x0 = rnd((rows, width), 1)
    pend_a, pend_b = rnd((rows, width), 2), rnd((rows, width), 3)

    class B:
        pass
    for t, entry in enumerate([first] + others):
        b = B()
        b.status = torch.zeros(1, dtype=torch.int32, device=DEV)
        b.per_step = {"embedding_rows": x0.to(DEV)}
        h = rnd((rows, width), 10 + t, 2.0)
        out, pending = entry.forward(h.to(DEV), ScaledSum(pend_a.to(DEV), pend_b.to(DEV)) if t else None, b)
        assert pending is None and b.status.item() == 0
        x = h.double() + ((pend_a.double() + pend_b.double()) if t else 0.0)
        want = torch.cat([x, x0.double()], dim=-1) @ w["lp.in"].T + w["lp.step"][t]
        close(out, want, "float32", t)
    with pytest.raises(ValueError):
        LoopEntry("lp.in", "lp.step", width, times, times)


# ------------------------------------------------------------------------------------------------ whole models

@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("sosuvik")
    return {name: ts.make_folder(tmp, raw, seed=i + 1) for i, (name, (raw, _)) in enumerate(ts.CONFIGS.items())}


_plain_memo = {}


def plain_logits(folder, raw, tokens):
    key = (folder, tuple(tokens))
    if key not in _plain_memo:
        _plain_memo[key] = plain.forward(raw, ts.weights(folder), tokens)
    return _plain_memo[key]


def clear_choices(folder, raw, tokens, least=0.03):
    """[T] bool: rows of which every routed layer run chooses its experts by a margin that bfloat16 rounding cannot turn.
    (Another expert changes a row by far more than rounding does; a row behind it reads that row's keys and moves a little.)"""
    margins = []
    plain.forward(raw, ts.weights(folder), tokens, margins_out=margins)
    ok = torch.ones(len(tokens), dtype=torch.bool)
    for m in margins:
        ok &= m > least
    return ok


def bfloat16_rows_agree(got, want, clear, bound, what):
    """Rows with clear choices within ``bound``; they are most rows; the others are not wild either."""
    err = ts.row_error(got, want)
    assert clear.float().mean().item() > 0.8, what
    assert err[clear].max().item() < bound and err.median().item() < 0.04, (what, int(err[clear].argmax()), err[clear].max().item(), err.median().item())
    assert err.max().item() < 1.2, what


def requests_for(raw, lengths, seed):
    return {f"q{i}": p for i, p in enumerate(tiny.prompts(raw["vocab"], lengths, seed=seed))}


WAYS = {"whole": replay.whole, "tail": lambda r: replay.tail_one_by_one(r, 40), "portions": replay.portions, "mixed": replay.mixed}
LENGTHS = {"S1": [150, 1, 2, 61, 34, 97], "S2": [260, 70, 1, 129, 3], "S3": [300, 3, 66, 2, 131], "S4": [120, 8, 2, 57]}


@pytest.mark.parametrize("name", ["S1", "S2", "S3", "S4"])
def test_float32_replay_every_way_against_the_plain_implementation(folders, name):
    from rust_mlx_b200.engine import Engine
    raw, page = ts.CONFIGS[name]
    reqs = requests_for(raw, LENGTHS[name], seed=11)
    want = {rid: plain_logits(folders[name], raw, toks) for rid, toks in reqs.items()}
    first = None
    for way, cut in WAYS.items():
        steps = cut(reqs)
        # a cache just large enough and four slots: pages are used again as requests end
        eng = Engine(folders[name], dtype="float32", max_tokens=replay.tokens_needed(steps, page), page_size=page, max_requests=4)
        got = replay.run_engine(eng, steps)
        eng.pools.table.check()
        assert eng.pools.table.live() == 0
        for rid in reqs:
            err = ts.row_error(got[rid], want[rid])
            assert err.max().item() < 2e-4, (name, way, rid, int(err.argmax()), err.max().item())
        if first is None:
            first = got
        else:       # the way of cutting changes a row by rounding at most
            for rid in reqs:
                assert ts.row_error(got[rid], first[rid]).max().item() < 2e-5, (name, way, rid)


@pytest.mark.parametrize("name", ["S1", "S2", "S3", "S4"])
def test_bfloat16_replay_every_way(folders, name):
    from rust_mlx_b200.engine import Engine
    raw, page = ts.CONFIGS[name]
    reqs = requests_for(raw, LENGTHS[name], seed=12)
    want = {rid: plain_logits(folders[name], raw, toks) for rid, toks in reqs.items()}
    clear = torch.cat([clear_choices(folders[name], raw, toks) for toks in reqs.values()])
    for way, cut in WAYS.items():
        steps = cut(reqs)
        eng = Engine(folders[name], dtype="bfloat16", max_tokens=replay.tokens_needed(steps, page), page_size=page, max_requests=4)
        got = replay.run_engine(eng, steps)
        eng.pools.table.check()
        bfloat16_rows_agree(torch.cat([got[rid] for rid in reqs]), torch.cat([want[rid] for rid in reqs]), clear, 0.15, (name, way))


def test_every_layer_run_against_the_plain_implementation(folders):
    """The stream after every layer run (a looped layer counts each time), in 32-bit: a difference is found at the first
    run that shows it.  The stream after run r is what the schedule's next block finds; a pass's entry finds it too."""
    from rust_mlx_b200.engine import Engine
    for name in ("S1", "S3", "S4"):
        raw, page = ts.CONFIGS[name]
        toks = tiny.prompts(raw["vocab"], [45], seed=5)[0]
        layers = []
        plain.forward(raw, ts.weights(folders[name]), toks, layers_out=layers)
        eng = Engine(folders[name], dtype="float32", max_tokens=128, page_size=page, max_requests=2)
        _, taken = eng.step_with_intermediates([("a", toks, [])], ["a"])
        runs = [i for i, call in enumerate(eng.spec.schedule) if call.cache is not None]      # (entries of passes hold no cache)
        assert len(runs) == len(layers) == len(plain.order_of_runs(raw))
        for r in range(len(runs) - 1):
            got = taken[f"run{runs[r] + 1}.residual"].double().cpu()
            assert (got - layers[r]).abs().max().item() < 1e-4 * (1 + layers[r].abs().max().item()), (name, r)


def needle_model(tmp_path, latent, chunk=None):
    """One layer whose mixer decides: scores spread so widely that single keys far back carry a row's weight."""
    mixer = ts.lat(2, 16, 8, 16, 24, scale=0.3) if latent else ts.attn(2, 1, 16, 16, ts.rot(1e4, 8), scale=0.3, chunk=chunk)
    raw = ts.model(90, 48, [ts.layer(mixer, None)])
    return raw, ts.make_folder(tmp_path, raw, seed=5, sharp=40.0, out_boost=30.0)


@pytest.mark.parametrize("latent", [False, True])
def test_far_keys_decide_and_are_found_in_prompts_and_in_decoding(tmp_path, latent):
    from rust_mlx_b200.engine import Engine
    raw, folder = needle_model(tmp_path, latent)
    toks = tiny.prompts(90, [520], seed=3)[0]
    want = plain.forward(raw, ts.weights(folder), toks)
    for cut in (replay.whole, lambda r: replay.tail_one_by_one(r, 60), replay.portions):
        steps = cut({"a": toks})
        eng = Engine(folder, dtype="float32", max_tokens=replay.tokens_needed(steps, 16), page_size=16, max_requests=2)
        got = replay.run_engine(eng, steps)["a"]
        assert ts.row_error(got, want).max().item() < 2e-4
    # the plain implementation itself, told to read its own chunk of 300 positions only, gives other logits: keys far
    # away carry weight
    s = plain.sees
    try:
        plain.sees = lambda T, chunk=None, start=0: s(T, 300, start)
        near = plain.forward(raw, ts.weights(folder), toks)
    finally:
        plain.sees = s
    assert ts.row_error(near[400:], want[400:]).max().item() > 0.05
    eng = Engine(folder, dtype="bfloat16", max_tokens=1024, page_size=16, max_requests=2)
    got = replay.run_engine(eng, replay.tail_one_by_one({"a": toks}, 60))["a"]
    err = ts.row_error(got, want)
    assert err.max().item() < 0.4 and err.median().item() < 0.08


@pytest.mark.parametrize("chunk, page", [(48, 16), (40, 64), (64, 64)])
def test_a_chunks_edge_shows_in_the_logits_of_prompts_and_decoded_tokens(tmp_path, chunk, page):
    """With scores this sharp a chunk that is one position off (a key too many, a key too few) changes the logits of the
    rows around every edge by far more than the bound; rows are taken whole, decoded and in small portions."""
    from rust_mlx_b200.engine import Engine
    raw, folder = needle_model(tmp_path, False, chunk=chunk)
    toks = tiny.prompts(90, [3 * chunk + 11], seed=chunk)[0]
    want = plain.forward(raw, ts.weights(folder), toks)
    s = plain.sees
    for off in (-1, 1):
        try:
            plain.sees = lambda T, c=None, start=0: s(T, c + off if c else c, start)
            wrong = plain.forward(raw, ts.weights(folder), toks)
        finally:
            plain.sees = s
        assert ts.row_error(wrong, want).max().item() > 0.05
    for dtype, bound in (("float32", 2e-4), ("bfloat16", 0.3)):
        for cut in (replay.whole, lambda r: replay.tail_one_by_one(r, 2 * chunk + 5), replay.portions):
            steps = cut({"a": toks})
            eng = Engine(folder, dtype=dtype, max_tokens=replay.tokens_needed(steps, page), page_size=page, max_requests=2)
            got = replay.run_engine(eng, steps)["a"]
            assert ts.row_error(got, want).max().item() < bound, (dtype, chunk)


def test_pages_that_are_used_again_give_the_same_bits(folders):
    """Two slots and pages for one long request: every request takes over what the one before it left (keys of another
    request, of another pass of the loop); the same request run again gives the same bits as in a fresh engine."""
    from rust_mlx_b200.engine import Engine
    raw, page = ts.CONFIGS["S1"]
    prompts = tiny.prompts(raw["vocab"], [70, 40, 70, 9], seed=9)
    fresh = []
    for p in prompts:
        eng = Engine(folders["S1"], dtype="float32", max_tokens=128, page_size=page, max_requests=2)
        half = len(p) // 2
        eng.step([("x", p[:half], [])])
        fresh.append(eng.step([("x", p[half:], list(range(len(p) - half)))], ["x"]).cpu())
    eng = Engine(folders["S1"], dtype="float32", max_tokens=128, page_size=page, max_requests=2)
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
    for name in ("S1", "S3"):
        raw, page = ts.CONFIGS[name]
        prompts = tiny.prompts(raw["vocab"], [140, 33, 2, 71], seed=17)
        for dtype, bound in (("float32", 2e-5), ("bfloat16", 0.08)):
            alone = []
            for p in prompts:
                eng = Engine(folders[name], dtype=dtype, max_tokens=256, page_size=page, max_requests=4)
                eng.step([("x", p[:-1], [])])
                alone.append(eng.step([("x", p[-1:], [0])], ["x"]).float().cpu())
            eng = Engine(folders[name], dtype=dtype, max_tokens=512, page_size=page, max_requests=4)
            eng.step([(0, prompts[0][:-1], []), (1, prompts[1][:-1], [])])
            # request 0 and 1 decode one token beside the whole of request 2 and a portion of request 3
            got = eng.step([(0, prompts[0][-1:], [0]), (2, prompts[2], [1]), (1, prompts[1][-1:], [0]), (3, prompts[3][:-1], [])], [0, 1, 2]).float().cpu()
            last = eng.step([(3, prompts[3][-1:], [0])], [3]).float().cpu()
            for row, i in ((got[0], 0), (got[1], 2), (got[2], 1), (last[0], 3)):
                assert ts.row_error(row[None], alone[i]).item() < bound, (name, dtype, i)


def test_long_decoding(folders):
    from rust_mlx_b200.engine import Engine
    raw, page = ts.CONFIGS["S1"]
    toks = tiny.prompts(raw["vocab"], [330], seed=21)[0]
    want = plain_logits(folders["S1"], raw, toks)
    eng = Engine(folders["S1"], dtype="float32", max_tokens=512, page_size=page, max_requests=2)
    got = replay.run_engine(eng, replay.tail_one_by_one({"a": toks}, 325))["a"]
    assert ts.row_error(got, want).max().item() < 2e-4


def greedy(raw, w, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(plain.forward(raw, w, ids)[-1].argmax()))
    return ids[len(prompt):]


def test_greedy_generation_through_the_scheduler(folders):
    from rust_mlx_b200.engine import Engine
    for name in ("S1", "S4"):
        raw, page = ts.CONFIGS[name]
        w = ts.weights(folders[name])
        prompts = tiny.prompts(raw["vocab"], [30, 3, 55, 9, 41], seed=31)
        want = [greedy(raw, w, p, 8) for p in prompts]
        # a cache too small for all five at once and three slots: requests wait, step back and are computed again
        eng = Engine(folders[name], dtype="float32", max_tokens=4 * page * 2 + 2 * page, page_size=page, max_requests=3)
        got = eng.generate(prompts, max_tokens=8, prefill_chunk=13, ignore_eos=True)
        assert got == want, name
        eng.pools.table.check()


def test_bfloat16_generation_in_graphs_equals_plain_launches(folders):
    from rust_mlx_b200.engine import Engine
    for name in ("S3", "S1"):
        raw, page = ts.CONFIGS[name]
        w = ts.weights(folders[name])
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
    raw, page = ts.CONFIGS["S1"]
    reqs = requests_for(raw, [40, 1, 77, 20, 5], seed=51)
    steps = replay.mixed(reqs)
    got = replay.run_trace_tool(folders["S1"], "float32", steps, str(tmp_path / "out"), replay.tokens_needed(steps, 64), raw["vocab"])
    for rid, toks in reqs.items():
        assert ts.row_error(got[rid], plain_logits(folders["S1"], raw, toks)).max().item() < 2e-4


def random_configuration(seed):
    """Sizes, constants, the order of layers and the loop drawn from a seed (every choice a model of this design may make)."""
    r = random.Random(seed)
    width = r.choice([48, 72, 96, 136])
    layers = []
    n = r.randint(2, 5)
    for _ in range(n):
        if r.random() < 0.5:
            kv = r.choice([1, 2, 3])
            heads = kv * r.choice([1, 2, 4])
            dim, vdim = r.choice([8, 16, 32, 64]), r.choice([8, 16, 24, 64])
            dims = r.choice([2, dim // 2, dim]) // 2 * 2
            scaling = r.choice([None, (r.choice([2.0, 8.0, 32.0]), r.choice([16, 64, 256]), r.choice([4.0, 32.0]), r.choice([1.0, 2.0]))])
            mixer = ts.attn(heads, kv, dim, vdim, ts.rot(r.choice([50.0, 1e4, 1e6]), dims, scaling), scale=r.uniform(0.1, 0.3),
                            softcap=r.choice([None, 2.0, 30.0]), chunk=r.choice([None, 5, 16, 33, 64, 100]))
        else:
            mixer = ts.lat(r.choice([1, 2, 3, 5]), r.choice([4, 8, 16, 32]), r.choice([2, 8, 16, 32]), r.choice([4, 8, 16, 32]),
                           r.choice([8, 16, 24, 40]), base=r.choice([50.0, 1e4]), scale=r.uniform(0.1, 0.3))
        if r.random() < 0.25:
            mlp = None
        else:
            count = r.choice([1, 2, 3, 4])
            per = r.choice([1, 2, 3])
            experts = count * per
            keep = r.randint(1, count)
            top = r.randint(1, keep * per)
            mlp = ts.moe(r.choice([8, 24, 64, 128]), experts, top, r.choice([0.2, 0.5, 7.0]), r.choice([1.0, 2.5]),
                         (count, keep) if count > 1 or r.random() < 0.5 else None)
        layers.append(ts.layer(mixer, mlp))
    loop = None
    if r.random() < 0.7:
        start = r.randint(0, n - 1)
        loop = (start, r.randint(start + 1, n), r.randint(1, 3))
    return ts.model(r.randint(50, 300), width, layers, loop=loop, eps=r.choice([1e-5, 1e-6]), logit_scale=r.choice([None, 0.5, 2.0]))


@pytest.mark.parametrize("seed", range(10))
def test_random_configurations_replayed_in_mixed_steps(tmp_path, seed):
    from rust_mlx_b200.engine import Engine
    raw = random_configuration(seed)
    folder = ts.make_folder(tmp_path, raw, seed=100 + seed)
    reqs = requests_for(raw, [70, 1, 33, 2, 90, 17], seed=seed)
    want = {rid: plain.forward(raw, ts.weights(folder), toks) for rid, toks in reqs.items()}
    clear = {rid: clear_choices(folder, raw, toks) for rid, toks in reqs.items()}
    page = [16, 32, 64][seed % 3]
    for dtype, bound in (("float32", 2e-4), ("bfloat16", 0.2)):
        for cut in (replay.mixed, replay.portions):
            steps = cut(reqs)
            eng = Engine(folder, dtype=dtype, max_tokens=replay.tokens_needed(steps, page), page_size=page, max_requests=4)
            got = replay.run_engine(eng, steps)
            eng.pools.table.check()
            for rid in reqs:
                err = ts.row_error(got[rid], want[rid])
                if dtype == "bfloat16":
                    err = err[clear[rid]]
                assert err.numel() == 0 or err.max().item() < bound, (seed, dtype, rid, int(err.argmax()), err.max().item(), raw)
            if dtype == "bfloat16":
                assert torch.cat(list(clear.values())).float().mean().item() > 0.3
