"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]

The default run has the layer sizes of Qwen3-8B with random weights in bfloat16: decode at
batch 8 from a context of 2,048 tokens per request.  It prints ONE JSON line.  ``value`` is
decoded tokens per second, timed on the device with CUDA events over exactly K steps (each
step: upload of the step's ids and tables from pinned memory, the model, greedy sampling).
``e2e`` is the same through the Python entry point (``Engine.generate``): host token ids in,
host token ids out, one host synchronisation per step; the ids it generated are then compared
with those of its warm-up run and of a run without graphs and in lockstep (``checked``), as
the reference's benchmarks compare every timed run's ids with the first run's
(src/bin/batch-bench.rs:147-151).  ``prefill`` is one 2,048-token prompt in one step;
``roofline`` is the decode step's bytes (every weight once plus the live requests' cache)
over its time.  Weights (15 GB) are far larger than L2, so no flush is needed between steps.

``--per-kernel`` instead times the phases of one decode step one by one (CUDA events between
the kernels, inside a captured graph, so without host gaps and without overlap between
neighbouring kernels) and prints bytes, time and fraction of the memory peak of each: a
synchronised diagnostic, not shares of the natural run time (the reference's
src/bin/profile.rs:22-36 does the same per phase).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], num_hidden_layers=36, hidden_size=4096,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
                vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
                max_position_embeddings=4096)
# the Qwen3-4B and Qwen3-32B layer sizes beside the default
SHAPES = {
    "qwen3-8b": QWEN3_8B,
    "qwen3-4b": dict(QWEN3_8B, hidden_size=2560, intermediate_size=9728, tie_word_embeddings=True),
    "qwen3-32b": dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600),
}
CONTEXT = 2048          # tokens each request holds when decoding starts
MAX_CONTEXT = 4096
PREFILL_TOKENS = 2048
PAGE = 64


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if os.path.exists(path):
        try:
            raw = json.load(open(path))
            out["hbm_gbs"] = float(raw.get("hbm_gbs", out["hbm_gbs"]))
            out["bf16_tflops"] = float(raw.get("bf16_tflops_sustained", raw.get("bf16_tflops", out["bf16_tflops"])))
            out["source"] = "measured"
        except Exception:
            pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def model_bytes(cfg, layers):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"] * h
    o = cfg["num_attention_heads"] * cfg["head_dim"] * h
    per_layer = qkv + o + 3 * h * i
    params = layers * per_layer + v * h           # the head once; embedding rows are a few KB
    return params * 2, per_layer, v * h


def kv_bytes_per_token(cfg, layers):
    return layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg, layers, tokens):
    _, per_layer, head = model_bytes(cfg, layers)
    gemm = 2.0 * tokens * layers * per_layer + 2.0 * head          # logits for the last row only
    attn = 2.0 * tokens * tokens * cfg["head_dim"] * cfg["num_attention_heads"] * layers   # causal: half of 4 T^2 d
    return gemm + attn


class DecodeRun:
    """B live requests holding CONTEXT tokens each (synthetic cache), stepped one token at a time."""

    def __init__(self, engine, batch, context):
        import torch
        self.e, self.batch, self.context, self.torch = engine, batch, context, torch
        self.rids = list(range(10_000, 10_000 + batch))
        self.len = context
        for r in self.rids:
            engine.pools.open(r)
            engine.pools.table.reserve(r, context)
            engine.pools.table.commit(r, context)
        g = torch.Generator().manual_seed(batch)
        self.ids = torch.randint(0, engine.vocab_size, (4096, batch), generator=g).tolist()
        self.out = torch.empty(batch, dtype=torch.int32, device=engine.device)
        self.n = 0

    def step(self):
        from rust_mlx_b200.engine.batch import SequenceInput, build_batch
        e = self.e
        for r in self.rids:
            e.pools.table.reserve(r, self.len + 1)
        toks = self.ids[self.n % len(self.ids)]
        seqs = [SequenceInput(r, self.len, [toks[i]], [0]) for i, r in enumerate(self.rids)]
        if e.graphs is not None:      # what generation does for a decode step: one captured graph
            e.graphs.run(seqs, None, None)
        else:
            batch = build_batch(seqs, e.pools, e.device, e._status, e.vocab_size)
            logits = e.forward(batch)
            e.ops.sample(logits, None, None, self.out)
        self.len += 1
        self.n += 1
        for r in self.rids:
            e.pools.table.commit(r, self.len)

    def close(self):
        for r in self.rids:
            self.e.pools.table.close(r)


def time_decode(engine, batch, steps, warmup, clocks=None):
    import torch
    from rust_mlx_b200.kernels import ops
    run = DecodeRun(engine, batch, CONTEXT)
    try:
        for _ in range(warmup):
            run.step()
        torch.cuda.synchronize()
        if clocks:
            clocks.start()
        launches0 = ops.launch_count
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            run.step()
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / steps
        engine.check_status()
        return ms, ops.launch_count - launches0, (clocks.stop() if clocks else None)
    finally:
        run.close()


def time_prefill(engine, tokens, reps=3, start_at=0):
    """One portion of ``tokens`` prompt tokens in one step, the request holding ``start_at`` tokens already (0: a whole
    prompt from its start; otherwise a later portion of a long prompt, its earlier keys being the synthetic cache)."""
    import torch
    from rust_mlx_b200.engine.batch import SequenceInput, build_batch
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, engine.vocab_size, (tokens,), generator=g).tolist()
    best = None
    for rep in range(reps + 1):
        rid = 20_000 + rep
        engine.pools.open(rid)
        if start_at:
            engine.pools.table.reserve(rid, start_at)
            engine.pools.table.commit(rid, start_at)
        engine.pools.table.reserve(rid, start_at + tokens)
        batch = build_batch([SequenceInput(rid, start_at, ids, [tokens - 1])], engine.pools, engine.device, engine._status,
                            engine.vocab_size)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        engine.forward(batch)
        stop.record()
        torch.cuda.synchronize()
        engine.pools.table.close(rid)
        ms = start.elapsed_time(stop)
        if rep > 0:                      # the first repetition warms up
            best = ms if best is None else min(best, ms)
    engine.check_status()
    return best


def time_e2e(engine, batch, new_tokens):
    """Through the Python entry point: prompts of CONTEXT host token ids, ``new_tokens`` generated each."""
    import torch
    g = torch.Generator().manual_seed(7)
    prompts = torch.randint(0, engine.vocab_size, (batch, CONTEXT), generator=g).tolist()
    opts = dict(ignore_eos=True, prefill_chunk=2048, max_batch_tokens=batch * CONTEXT)
    # warm-up with the same shapes: the decode step of this batch size is captured into its graph here
    warm = engine.generate(prompts, max_tokens=3, **opts)
    r = engine.generate_detailed(prompts, max_tokens=new_tokens, **opts)
    decoded = r.generated_tokens - batch
    # what was generated: the timed run's ids begin with the warm-up run's, and a run of plain launches in
    # lockstep (no graphs, no step launched ahead) generates the same ids
    graphs, engine.graphs = engine.graphs, None
    try:
        plain = engine.generate(prompts, max_tokens=new_tokens, run_ahead=False, **opts)
    finally:
        engine.graphs = graphs
    checked = all(len(t) == new_tokens for t in r.tokens) and all(t[:3] == w for t, w in zip(r.tokens, warm)) and plain == r.tokens
    if not checked:
        first = next(((i, j) for i, (x, y) in enumerate(zip(r.tokens, plain)) for j, (u, v) in enumerate(zip(x, y)) if u != v), None)
        print(f"bench.py: the timed run's ids differ from the check runs' (first difference at request, token {first})",
              file=sys.stderr)
    # bytes per decode step: ids, positions, sequence indices, starts, lengths, slots, rows, block tables up; tokens + status down
    # a captured decode step uploads one buffer of fixed layout: ids, positions, sequence indices, starts, lengths,
    # slots, rows, temperatures, uniforms and block tables of the context limit
    from rust_mlx_b200.engine.batch import BatchLayout
    from rust_mlx_b200.engine.graphs import bucket
    b = bucket(batch)
    h2d = 4 * BatchLayout(b, b, b, [engine.max_context // PAGE for _ in engine.pools.paged_groups]).total
    d2h = 4 * (b + 1)
    return decoded / r.decode_seconds, h2d, d2h, checked


def per_kernel(engine, raw, a, pk):
    """One decode step of ``a.batch`` requests at CONTEXT tokens, captured with an event after every phase of every
    layer; replayed ``a.steps`` times.  Prints a table (standard error) and one JSON line."""
    import torch
    from rust_mlx_b200.engine.batch import SequenceInput, build_batch
    run = DecodeRun(engine, a.batch, CONTEXT)
    try:
        e = engine
        for r in run.rids:
            e.pools.table.reserve(r, run.len + 1)
        seqs = [SequenceInput(r, run.len, [run.ids[0][i]], [0]) for i, r in enumerate(run.rids)]
        batch = build_batch(seqs, e.pools, e.device, e._status, e.vocab_size)
        out = torch.empty(a.batch, dtype=torch.int32, device=e.device)
        marks = []          # (phase that ended here, event)

        def tap(name, tensor):
            ev = torch.cuda.Event(enable_timing=True, external=True)
            ev.record()
            marks.append((name, ev))

        def step():
            marks.clear()
            tap("start", None)
            tap("nothing", None)          # two events with no kernel between them: what an event itself costs
            logits = e.forward(batch)
            e.ops.sample(logits, None, None, out)
            tap("head", None)
        e.forward(batch)                      # buffers reach their size
        torch.cuda.synchronize()
        e._ctx.tap = tap
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
        finally:
            e._ctx.tap = None
        # what ends at a mark, by the mark's name: the kernels between it and the mark before
        phase = {"residual": None, "norm1": "add + norm", "qkv": "q/k/v product", "q_rot": "norm + rotation + cache write",
                 "attn_out": "attention", "mixer_out": "output product", "norm2": "add + norm", "ffn_act": "gate/up product + SwiGLU",
                 "ffn_out": "down product", "head": "final norm + head + sampling", "nothing": "(an event alone)"}
        total = {}
        for _ in range(max(a.warmup, 3)):
            graph.replay()
        for _ in range(a.steps):
            graph.replay()
            torch.cuda.synchronize()
            last = marks[0][1]
            for name, ev in marks[1:]:
                if phase.get(name) is None:
                    continue            # (the stream before a block's norm: the same place as its norm1 mark)
                total.setdefault(phase[name], []).append(last.elapsed_time(ev) * 1e3)
                last = ev
        h, inter, v = raw["hidden_size"], raw["intermediate_size"], raw["vocab_size"]
        nq, nkv, hd, layers = raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"], a.layers
        per_layer_bytes = {"q/k/v product": (nq + 2 * nkv) * hd * h * 2, "output product": nq * hd * h * 2,
                           "gate/up product + SwiGLU": 2 * inter * h * 2, "down product": inter * h * 2,
                           "attention": a.batch * (CONTEXT + 1) * 2 * nkv * hd * 2,
                           "add + norm": a.batch * h * (4 + 4 + 2 + 2), "norm + rotation + cache write": a.batch * (nq + 2 * nkv) * hd * 4,
                           "final norm + head + sampling": v * h * 2 + a.batch * v * 8}
        rows, step_us = [], 0.0
        event_us = sum(total.pop("(an event alone)")) / a.steps      # subtracted from every phase below
        for name, times in total.items():
            calls = len(times) // a.steps
            us = max(sum(times) / a.steps / calls - event_us, 0.01)
            gbs = per_layer_bytes[name] / us / 1e3
            step_us += us * calls
            rows.append({"phase": name, "calls_per_step": calls, "us": round(us, 2), "bytes": per_layer_bytes[name],
                         "gb_per_s": round(gbs, 1), "frac": round(gbs / pk["hbm_gbs"], 3)})
        print(f"{'phase':34s} {'calls':>5s} {'us each':>9s} {'MB each':>9s} {'GB/s':>8s} {'of peak':>8s}", file=sys.stderr)
        for r_ in rows:
            print(f"{r_['phase']:34s} {r_['calls_per_step']:5d} {r_['us']:9.2f} {r_['bytes'] / 1e6:9.2f} {r_['gb_per_s']:8.1f} {r_['frac']:8.3f}",
                  file=sys.stderr)
        print(f"(an event alone: {event_us:.2f} us, subtracted from every phase)", file=sys.stderr)
        print(json.dumps({"per_kernel": rows, "step_us_serialised": round(step_us, 1), "event_us": round(event_us, 2), "batch": a.batch, "context": CONTEXT,
                          "layers": layers, "shape": a.shape, "peak_gb_per_s": pk["hbm_gbs"], "of": pk["source"],
                          "note": "events between kernels inside one captured graph: no host gaps, no overlap of neighbours"}))
        return 0
    finally:
        run.close()


def continuous(cfg, raw, a):
    """64 requests, prompts of 128..3072 uniform-random ids, 256 generated tokens each, through the scheduler:
    portions of prompts (at most 512 tokens a step) run beside the decoded tokens of the requests already past theirs."""
    import random

    import torch
    from rust_mlx_b200.engine import Engine
    rng = random.Random(0)
    lengths = [rng.randrange(128, 3073) for _ in range(64)]
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, raw["vocab_size"], (n,), generator=g).tolist() for n in lengths]
    new_tokens = 256
    cache_tokens = sum(-(-(n + new_tokens) // PAGE) * PAGE for n in lengths)
    engine = Engine(cfg, dtype="bfloat16", random_weights=True, seed=0, max_tokens=cache_tokens, page_size=PAGE, max_requests=64,
                    tuning=a.policy)
    opts = dict(max_tokens=new_tokens, ignore_eos=True, prefill_chunk=512, max_batch_tokens=512 + 64, max_seqs=64)
    engine.generate(prompts[:8], **dict(opts, max_tokens=8))            # warm-up: kernels, graphs of the first sizes
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    r = engine.generate_detailed(prompts, **opts)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    line = {"metric": "continuous batching: generated tok/s over the whole run", "value": round(r.generated_tokens / wall, 1),
            "unit": "tok/s", "impl": "ours", "n_gpus": 1, "dtype": "bf16", "data": "synthetic",
            "config": {"model": a.shape + " shape, random weights", "layers": a.layers, "requests": 64, "prompt_tokens": r.prompt_tokens,
                       "generated_tokens": r.generated_tokens, "prefill_chunk": 512, "max_batch_tokens": 576, "page_size": PAGE},
            "seconds": round(wall, 3), "steps": r.steps, "preemptions": r.preemptions,
            "total_tok_per_s": round((r.generated_tokens + r.prompt_tokens) / wall, 1)}
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------------------------------------
# --family resolorn: the Resolorn design at layer sizes of real models, beside the Qwen3 dense decoder of equal
# width, depth, head size and feed-forward width: decode and prefill throughput, and every phase of a step against
# its roofline (bytes over the measured copy bandwidth, or flops over the measured product peak, whichever is slower).

def _latent_mixer(heads, dim, vdim, q_rank, kv_rank, window=0, kv_from=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": dim ** -0.5}
    if window:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def resolorn_shape(width, heads, dim, q_rank, kv_rank, ff, experts, top, expert_ff, shared_ff, vocab, window, groups=1):
    """Groups of four layers: dense and routed feed-forwards in turn; the second pair reads the latents of the first
    routed layer; the first and third have a window."""
    layers = []
    for g in range(groups):
        base = 4 * g
        dense = {"kind": "dense", "ff": ff}
        moe = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top}, "shared": {"ff": shared_ff}}
        layers += [{"type": "latent_attention", "mixer": _latent_mixer(heads, dim, dim, q_rank, kv_rank, window), "mlp": dense},
                   {"type": "latent_attention", "mixer": _latent_mixer(heads, dim, dim, q_rank, kv_rank), "mlp": moe},
                   {"type": "latent_attention", "mixer": _latent_mixer(heads, dim, dim, q_rank, kv_rank, window, kv_from=base + 1), "mlp": dense},
                   {"type": "latent_attention", "mixer": _latent_mixer(heads, dim, dim, q_rank, kv_rank, kv_from=base + 1), "mlp": moe}]
    return {"architecture": "Resolorn", "vocab": vocab, "width": width, "max_positions": 2 * MAX_CONTEXT, "norm": {"eps": 1e-6},
            "residual_mult": 0.5, "layers": layers}


FAMILY_SIZES = {
    # width, heads, dim, q_rank, kv_rank, dense ff, experts, top, expert ff, shared ff, vocab, window
    "2k": dict(width=2048, heads=16, dim=64, q_rank=512, kv_rank=128, ff=8192, experts=32, top=4, expert_ff=1024, shared_ff=1024,
               vocab=32768, window=1024),
    "4k": dict(width=4096, heads=16, dim=128, q_rank=1536, kv_rank=128, ff=12288, experts=64, top=6, expert_ff=1408, shared_ff=2816,
               vocab=65536, window=1024),
}


# --family gugalorn: the Gugalorn design (state-space layers and layers of softmax attention beside gated linear attention)
# at layer sizes of real models, beside the Qwen3 dense decoder of equal width, depth, heads and feed-forward width.

def gugalorn_shape(width, heads, kv_heads, dim, rot, ssm_heads, ssm_vdim, state, ssm_groups, gla_heads, gla_dim, gla_vdim, ff, vocab,
                   groups=1):
    """Groups of four layers: a state-space layer without a feed-forward, two parallel layers with one, a state-space layer."""
    ssm = {"type": "mamba2", "mixer": {"heads": ssm_heads, "vdim": ssm_vdim, "state": state, "groups": ssm_groups, "conv": 4,
                                       "norm_groups": ssm_groups}, "mlp": None}
    par = {"type": "parallel",
           "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "rot": {"dims": rot, "base": 1e6}, "scale": dim ** -0.5},
                     "right": {"heads": gla_heads, "dim": gla_dim, "vdim": gla_vdim}, "left_scale": 1.0, "right_scale": 1.0},
           "mlp": {"kind": "dense", "ff": ff}}
    return {"architecture": "Gugalorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "canon": {"taps": 4}, "layers": [ssm, par, par, ssm] * groups}


GUGALORN_SIZES = {
    "2k": dict(width=2048, heads=16, kv_heads=4, dim=64, rot=32, ssm_heads=64, ssm_vdim=64, state=128, ssm_groups=8, gla_heads=16,
               gla_dim=128, gla_vdim=128, ff=8192, vocab=32768),
    "4k": dict(width=4096, heads=32, kv_heads=8, dim=128, rot=64, ssm_heads=128, ssm_vdim=64, state=128, ssm_groups=8, gla_heads=32,
               gla_dim=128, gla_vdim=128, ff=12288, vocab=65536),
}


def gugalorn_costs(raw, starts, counts):
    """tap name -> function(layer) -> (bytes, flops on the tensor cores) of the kernels that end at that tap."""
    n, W, S = sum(counts), raw["width"], len(counts)
    cached = sum(s + c for s, c in zip(starts, counts))

    def ssm(f):
        m = f["mixer"]
        inner = m["heads"] * m["vdim"]
        return m, inner, inner + 2 * m["groups"] * m["state"]

    def left(f):
        a = f["mixer"]["left"]
        return a["heads"], a["kv_heads"], a["dim"], a["vdim"]

    def right(f):
        g = f["mixer"]["right"]
        return g["heads"] * g["dim"], g["heads"] * g["vdim"], g["heads"] * g["dim"] * g["vdim"]

    return {
        "norm1": lambda f: (n * W * 12.0, 0.0), "norm2": lambda f: (n * W * 12.0, 0.0),
        "conv_in": lambda f: (n * W * 4.0, 0.0),
        "ssm_in": lambda f: _product(n, 2 * ssm(f)[1] + 2 * ssm(f)[0]["groups"] * ssm(f)[0]["state"] + ssm(f)[0]["heads"], W),
        "ssm_conv": lambda f: (4.0 * n * ssm(f)[2], 0.0),
        "recurrence_out": lambda f: (2.0 * n * ssm(f)[2] + 4.0 * n * ssm(f)[1] + 8.0 * S * ssm(f)[1] * ssm(f)[0]["state"], 0.0),
        "recurrence_normed": lambda f: (8.0 * n * ssm(f)[1], 0.0),
        "mixer_out": lambda f: _product(n, W, ssm(f)[1]),
        "qkv": lambda f: _product(n, (left(f)[0] + left(f)[1]) * (left(f)[2] + left(f)[3]), W),
        "q_rot": lambda f: (4.0 * n * (left(f)[0] + 2 * left(f)[1]) * left(f)[2], 0.0),
        "attn_out": lambda f: (4.0 * cached * left(f)[1] * left(f)[2] + 4.0 * n * left(f)[0] * left(f)[2],
                               4.0 * _keys_seen(starts, counts, 0) * left(f)[0] * left(f)[2]),
        "attn_gated": lambda f: (6.0 * n * left(f)[0] * left(f)[3], 0.0),
        "attn_proj": lambda f: _product(n, W, left(f)[0] * left(f)[3]),
        "gla_in": lambda f: _product(n, 2 * right(f)[0] + right(f)[1], W),
        "gla_recurrence_out": lambda f: (2.0 * n * (2 * right(f)[0] + right(f)[1]) + 4.0 * n * right(f)[1] + 8.0 * S * right(f)[2], 0.0),
        "gla_normed": lambda f: (6.0 * n * right(f)[1], 0.0),
        "gla_proj": lambda f: _product(n, W, right(f)[1]),
        "ffn_act": lambda f: _product(n, 2 * f["mlp"]["ff"], W),
        "ffn_out": lambda f: _product(n, W, f["mlp"]["ff"]),
    }


GUGALORN_PHASES = {"norm1": "add + norm", "norm2": "add + norm", "conv_in": "input convolution", "ssm_in": "state-space input product",
                   "ssm_conv": "inner convolution + silu", "recurrence_out": "state-space recurrence",
                   "recurrence_normed": "gate + group norm", "mixer_out": "state-space output product",
                   "qkv": "q/k/v/gate product", "q_rot": "whole-projection norm + rotation + cache write", "attn_out": "attention with a sink",
                   "attn_gated": "output gate", "attn_proj": "attention output product", "gla_in": "linear attention's q/f/v product",
                   "gla_recurrence_out": "gated linear recurrence", "gla_normed": "norm a head", "gla_proj": "linear attention's output product",
                   "ffn_act": "gate/up product + activation", "ffn_out": "down product"}


# --family sosuvik: the Sosuvik design (chunked attention with a sink and capped scores, attention through a latent with a
# rotated key part, experts chosen among groups, a looped layer) at layer sizes of real models, beside the Resolorn design
# (its closest relative here: latents and routed experts) and the Qwen3 dense decoder (whose attention kernels its
# attention layers run on) of equal width, depth, heads and latent row.

def sosuvik_shape(width, heads, kv_heads, dim, rot, kv_rank, rot_dim, experts, top, expert_ff, route_groups, keep, vocab, chunk, groups=1):
    """Four layer runs a group: attention whose chunk is longer than any context here, a latent layer, (in the first
    group the same latent layer again: a loop of two passes; elsewhere a second one), attention in chunks of ``chunk``."""
    scaling = {"factor": 4.0, "original": 8192, "fast": 16.0, "slow": 2.0}
    mlp = {"kind": "moe", "expert": {"ff": expert_ff, "limit": 7.0},
           "router": {"experts": experts, "top": top, "scale": 2.0, "groups": {"count": route_groups, "keep": keep}}}

    def attention(size):
        return {"type": "attention", "mlp": mlp,
                "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "softcap": 30.0,
                          "rot": {"base": 1e6, "dims": rot, "scaling": scaling}, "mask": {"size": size}}}
    latent = {"type": "latent_attention", "mlp": mlp,
              "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": dim, "kv_rank": kv_rank, "scale": (dim + rot_dim) ** -0.5,
                        "rot": {"base": 1e4, "dims": rot_dim}}}
    layers = [attention(4 * MAX_CONTEXT), latent, attention(chunk)]
    for _ in range(groups - 1):
        layers += [attention(4 * MAX_CONTEXT), latent, latent, attention(chunk)]
    return {"architecture": "Sosuvik", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "logit_scale": 0.25,
            "loop": {"start": 1, "stop": 2, "times": 2}, "layers": layers}


SOSUVIK_SIZES = {
    "2k": dict(width=2048, heads=16, kv_heads=4, dim=64, rot=32, kv_rank=112, rot_dim=16, experts=32, top=4, expert_ff=1024, route_groups=4,
               keep=2, vocab=32768, chunk=1024),
    "4k": dict(width=4096, heads=16, kv_heads=4, dim=128, rot=64, kv_rank=112, rot_dim=16, experts=64, top=6, expert_ff=1408, route_groups=8,
               keep=4, vocab=65536, chunk=1024),
}


def _keys_in_chunks(starts, counts, chunk):
    """(keys the step's tokens see, keys that are read at least once): a token reads its own chunk of positions up to itself."""
    seen = read = 0
    for s, c in zip(starts, counts):
        for p in range(s, s + c):
            seen += p % chunk + 1 if chunk else p + 1
        first = (s // chunk) * chunk if chunk else 0
        read += s + c - first
    return seen, read


def sosuvik_costs(raw, starts, counts):
    """tap name -> function(layer) -> (bytes, flops) of the kernels that end at that tap, or None where none ran."""
    n, W = sum(counts), raw["width"]
    everything = sum(s + c for s, c in zip(starts, counts))

    def kind(att, lat=None, loop=None):
        def cost(layer):
            f = {"attention": att, "latent_attention": lat, "loop": loop}[layer["type"]]
            return f(layer["mixer"]) if f is not None and layer["type"] != "loop" else (f() if f is not None else None)
        return cost

    def mlp(f):
        return lambda layer: f(layer["mlp"]) if layer.get("mlp") else None

    def touched(f):
        e, top = f["router"]["experts"], f["router"]["top"]
        return e * (1.0 - (1.0 - top / e) ** n)

    def row(m):
        need = m["kv_rank"] + m["rot_dim"]
        return next((s for s in (16, 32, 64, 96, 128) if s >= need), -(-need // 16) * 16)

    def chunked(m):
        seen, read = _keys_in_chunks(starts, counts, (m.get("mask") or {}).get("size", 0))
        return (2.0 * read * m["kv_heads"] * (m["dim"] + m["vdim"]) + 4.0 * n * m["heads"] * m["dim"],
                2.0 * seen * m["heads"] * (m["dim"] + m["vdim"]))

    return {
        # (both norms of a layer come from one kernel: stream 4 + 4, two pending terms, two normed rows)
        "norm1": kind(lambda m: (n * W * 16.0, 0.0), lambda m: (n * W * 16.0, 0.0)),
        "loop_in": kind(None, None, lambda: (n * W * 14.0, 0.0)),
        "loop_out": kind(None, None, lambda: (2.0 * (2 * W * W + 2 * n * W) + 8.0 * n * W, 4.0 * n * W * W)),
        "qkv": kind(lambda m: _product(n, m["heads"] * m["dim"] + m["kv_heads"] * (m["dim"] + m["vdim"]), W)),
        "q_rot": kind(lambda m: (4.0 * n * (m["heads"] * m["dim"] + m["kv_heads"] * (m["dim"] + m["vdim"])), 0.0)),
        "attn_proj": kind(lambda m: _product(n, W, m["heads"] * m["vdim"])),
        "latent_down": kind(None, lambda m: _product(n, m["heads"] * (m["dim"] + m["rot_dim"]) + m["kv_rank"] + m["rot_dim"], W)),
        # (a product a head into the latent's space, then norm + rotation + cache write)
        "q_latent": kind(None, lambda m: (2.0 * m["heads"] * (m["dim"] * m["kv_rank"] + n * (m["dim"] + m["kv_rank"]))
                                          + 2.0 * n * (m["kv_rank"] + m["rot_dim"] + row(m) + 2 * m["heads"] * m["rot_dim"]),
                                          2.0 * n * m["heads"] * m["dim"] * m["kv_rank"])),
        "attn_out": kind(chunked, lambda m: (2.0 * everything * row(m) + 4.0 * n * m["heads"] * row(m),
                                             4.0 * _keys_seen(starts, counts, 0) * m["heads"] * row(m))),
        "attn_values": kind(None, lambda m: (2.0 * m["heads"] * (m["vdim"] * m["kv_rank"] + n * (m["vdim"] + m["kv_rank"])),
                                             2.0 * n * m["heads"] * m["vdim"] * m["kv_rank"])),
        "mixer_out": kind(None, lambda m: _product(n, W, m["heads"] * m["vdim"])),
        "moe_ids": mlp(lambda f: (4.0 * f["router"]["experts"] * W + 2.0 * n * W, 0.0)),
        "moe_sorted": mlp(lambda f: (12.0 * n * f["router"]["top"], 0.0)),
        "moe_rows": mlp(lambda f: (4.0 * n * f["router"]["top"] * W, 0.0)),
        "moe_act": mlp(lambda f: (2.0 * (touched(f) * 2 * f["expert"]["ff"] * W + n * f["router"]["top"] * (W + f["expert"]["ff"])),
                                  2.0 * n * f["router"]["top"] * 2 * f["expert"]["ff"] * W)),
        "moe_expert_out": mlp(lambda f: (2.0 * (touched(f) * f["expert"]["ff"] * W + n * f["router"]["top"] * (W + f["expert"]["ff"])),
                                         2.0 * n * f["router"]["top"] * f["expert"]["ff"] * W)),
        "ffn_out": mlp(lambda f: (2.0 * n * W * (f["router"]["top"] + 1), 0.0)),
    }


SOSUVIK_PHASES = {"norm1": "add + two norms", "loop_in": "stream beside the embedding's rows", "loop_out": "loop entry product + step vector",
                  "qkv": "q/k/v product", "q_rot": "rotation + cache write",
                  "attn_out": lambda layer: "attention in chunks, capped, with a sink" if layer["type"] == "attention" else "attention over latents",
                  "attn_proj": "attention output product",
                  "latent_down": "query and latent down product", "q_latent": "queries into the latent's space + norm + rotation + cache write",
                  "attn_values": "values out of the latent's space (a product a head)", "mixer_out": "output product",
                  "moe_ids": "router among groups", "moe_sorted": "grouping by expert", "moe_rows": "rows into the experts' order",
                  "moe_act": "experts' gate/up products + clamped swish", "moe_expert_out": "experts' down products",
                  "ffn_out": "weighted sum of the experts"}


# --family reverax: the Reverax design (attention whose scores are mixed over the heads; windowed attention with turned values
# and learned sinks beside linear attention with a learned decay; norms in groups with scale vectors; dense feed-forwards and
# experts without a gate) at layer sizes of real models, beside the Gugalorn design (its closest relative here: softmax
# attention beside a linear recurrence) and the Qwen3 dense decoder of equal width, depth, heads and feed-forward width.

def reverax_shape(width, heads, kv_heads, dim, rot, right_heads, right_dim, rank, ff, experts, top, expert_ff, vocab, window, groups=1):
    """Four layers a group: mixed-score attention with a dense feed-forward, a parallel layer with experts, the same layer's
    tensors again with caches of their own, mixed-score attention with experts."""
    moe = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top}}
    att = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "rot": {"base": 1e6, "dims": rot}}
    side = {"left": dict(att, softcap=50.0, mask={"size": window}, rot={"base": 1e6, "dims": rot}),
            "right": {"heads": right_heads, "dim": right_dim, "rank": rank}, "left_scale": 1.0, "right_scale": 0.5}
    layers = []
    for g in range(groups):
        layers += [{"type": "attention", "mixer": att, "mlp": {"kind": "dense", "ff": ff}}, {"type": "parallel", "mixer": side, "mlp": moe},
                   {"type": "parallel", "mixer": side, "mlp": moe, "weights_of": 4 * g + 1}, {"type": "attention", "mixer": att, "mlp": moe}]
    return {"architecture": "Reverax", "vocab": vocab, "width": width, "norm": {"eps": 1e-6, "groups": 4}, "logit_scale": 0.5, "layers": layers}


REVERAX_SIZES = {
    "2k": dict(width=2048, heads=16, kv_heads=4, dim=64, rot=32, right_heads=32, right_dim=64, rank=64, ff=8192, experts=32, top=4,
               expert_ff=1024, vocab=32768, window=1024),
    "4k": dict(width=4096, heads=16, kv_heads=4, dim=128, rot=64, right_heads=64, right_dim=64, rank=64, ff=12288, experts=64, top=6,
               expert_ff=1408, vocab=65536, window=1024),
}


def reverax_costs(raw, starts, counts):
    """tap name -> function(layer) -> (bytes, flops on the tensor cores) of the kernels that end at that tap, or None."""
    n, W, S = sum(counts), raw["width"], len(counts)
    everything = sum(s + c for s, c in zip(starts, counts))

    def att(layer):
        return layer["mixer"] if layer["type"] == "attention" else layer["mixer"]["left"]

    def side(f):
        return lambda layer: f(layer["mixer"]["right"]) if layer["type"] == "parallel" else None

    def mlp(kind, f):
        return lambda layer: f(layer["mlp"]) if (layer.get("mlp") or {}).get("kind") == kind else None

    def touched(f):
        e, top = f["router"]["experts"], f["router"]["top"]
        return e * (1.0 - (1.0 - top / e) ** n)

    def attention(layer):
        m = att(layer)
        window = (m.get("mask") or {}).get("size", 0)
        read = sum(min(s + c, window + c) if window else s + c for s, c in zip(starts, counts))
        return (2.0 * read * m["kv_heads"] * (m["dim"] + m["vdim"]) + 4.0 * n * m["heads"] * m["dim"],
                2.0 * _keys_seen(starts, counts, window) * m["heads"] * (m["dim"] + m["vdim"]))

    def inner(r):
        return r["heads"] * r["dim"]

    def last(layer):
        f = layer.get("mlp") or {}
        if f.get("kind") == "dense":
            return _product(n, W, f["ff"])
        return (2.0 * n * W * (f["router"]["top"] + 1), 0.0) if f else None

    return {
        # (both norms of a layer come from one kernel: stream 4 + 4, up to three pending terms, two normed rows)
        "norm1": lambda layer: (n * W * 18.0, 0.0),
        "qkv": lambda layer: _product(n, att(layer)["heads"] * att(layer)["dim"] + att(layer)["kv_heads"] * (att(layer)["dim"] + att(layer)["vdim"]), W),
        "q_rot": lambda layer: (4.0 * n * (att(layer)["heads"] * att(layer)["dim"] + att(layer)["kv_heads"] * (att(layer)["dim"] + att(layer)["vdim"])), 0.0),
        "attn_out": attention,
        "attn_turned_back": lambda layer: (4.0 * n * att(layer)["heads"] * att(layer)["vdim"], 0.0),
        "attn_proj": lambda layer: _product(n, W, att(layer)["heads"] * att(layer)["vdim"]),
        "shift_mixes": side(lambda r: (12.0 * n * W, 0.0)),
        # (five products of the mixes and the decay's second small product)
        "decay_in": side(lambda r: (2.0 * (4 * inner(r) * W + r["rank"] * (W + inner(r)) + n * (5 * W + 5 * inner(r) + 2 * r["rank"])),
                                    2.0 * n * (4 * inner(r) * W + r["rank"] * (W + inner(r))))),
        "decay_recurrence_out": side(lambda r: (2.0 * n * 4 * inner(r) + 4.0 * n * inner(r) + 8.0 * S * inner(r) * r["dim"], 0.0)),
        "decay_normed": side(lambda r: (8.0 * n * inner(r), 0.0)),
        "decay_proj": side(lambda r: _product(n, W, inner(r))),
        "ffn_act": mlp("dense", lambda f: _product(n, 2 * f["ff"], W)),
        "moe_ids": mlp("moe", lambda f: (4.0 * f["router"]["experts"] * W + 2.0 * n * W, 0.0)),
        "moe_sorted": mlp("moe", lambda f: (12.0 * n * f["router"]["top"], 0.0)),
        "moe_rows": mlp("moe", lambda f: (4.0 * n * f["router"]["top"] * W, 0.0)),
        "moe_act": mlp("moe", lambda f: (2.0 * (touched(f) * f["expert"]["ff"] * W + n * f["router"]["top"] * (W + f["expert"]["ff"])),
                                         2.0 * n * f["router"]["top"] * f["expert"]["ff"] * W)),
        "moe_expert_out": mlp("moe", lambda f: (2.0 * (touched(f) * f["expert"]["ff"] * W + n * f["router"]["top"] * (W + f["expert"]["ff"])),
                                                2.0 * n * f["router"]["top"] * f["expert"]["ff"] * W)),
        "ffn_out": last,
    }


REVERAX_PHASES = {"norm1": "add (scale vectors) + two norms in groups", "qkv": "q/k/v product",
                  "q_rot": lambda layer: "bias + rotation + cache write" if layer["type"] == "attention" else "bias + head norms + rotation of q, k and v + cache write",
                  "attn_out": lambda layer: "attention with scores mixed over the heads" if layer["type"] == "attention" else "attention in a window, capped, with learned sinks",
                  "attn_turned_back": "results turned back", "attn_proj": "attention output product",
                  "shift_mixes": "token-shift mixes", "decay_in": "products of the mixes (r, k, v, g, decay)",
                  "decay_recurrence_out": "recurrence with a learned decay", "decay_normed": "norm a head + gate",
                  "decay_proj": "linear attention's output product", "ffn_act": "gate/up product + activation",
                  "moe_ids": "router (sigmoid scores)", "moe_sorted": "grouping by expert", "moe_rows": "rows into the experts' order, weighted",
                  "moe_act": "experts' up products + squared relu", "moe_expert_out": "experts' down products"}


def _product(n, rows, cols):
    """(bytes, flops) of [n, cols] . [rows, cols]^T in bfloat16."""
    return 2.0 * (rows * cols + n * cols + n * rows), 2.0 * n * rows * cols


def _keys_seen(starts, counts, window):
    """Sum over the step's tokens of the keys each sees (itself and those before it, inside its window)."""
    total = 0
    for s, c in zip(starts, counts):
        for p in range(s, s + c):
            total += min(p + 1, window) if window else p + 1
    return total


def resolorn_costs(raw, starts, counts):
    """tap name -> function(layer) -> (bytes, flops) of the kernels that end at that tap, for a step whose sequences hold
    ``starts`` tokens and bring ``counts`` more."""
    n, W = sum(counts), raw["width"]

    def cached(layer):      # latents read: every sequence's visible keys once (all heads share them)
        window = (layer["mixer"].get("mask") or {}).get("size", 0)
        return sum(min(s + c, window + c - 1) if window else s + c for s, c in zip(starts, counts))

    def mix(f):
        return lambda layer: f(layer["mixer"], layer)

    def mlp(f):
        return lambda layer: f(layer["mlp"], layer)

    def touched(f):         # experts whose weights a step reads, if rows choose uniformly
        e, top = f["router"]["experts"], f["router"]["top"]
        return e * (1.0 - (1.0 - top / e) ** n)

    return {
        "norm1": lambda layer: (n * W * 14.0, 0.0),
        "latent_down": mix(lambda m, layer: _product(n, m["q_rank"] + (0 if "kv_from" in m else m["kv_rank"]) + m["heads"], W)),
        "latent_q": mix(lambda m, layer: (4.0 * n * (m["q_rank"] + (0 if "kv_from" in m else m["kv_rank"])), 0.0)),
        "q_heads": mix(lambda m, layer: _product(n, m["heads"] * m["dim"], m["q_rank"])),
        "q_latent": mix(lambda m, layer: (2.0 * m["heads"] * (m["dim"] * m["kv_rank"] + n * (m["dim"] + m["kv_rank"])),
                                          2.0 * n * m["heads"] * m["dim"] * m["kv_rank"])),
        "attn_out": mix(lambda m, layer: (2.0 * cached(layer) * m["kv_rank"] + 4.0 * n * m["heads"] * m["kv_rank"],
                                          4.0 * _keys_seen(starts, counts, (m.get("mask") or {}).get("size", 0)) * m["heads"] * m["kv_rank"])),
        "attn_values": mix(lambda m, layer: (2.0 * m["heads"] * (m["vdim"] * m["kv_rank"] + n * (m["vdim"] + m["kv_rank"])),
                                             2.0 * n * m["heads"] * m["vdim"] * m["kv_rank"])),
        "attn_heads": mix(lambda m, layer: (4.0 * n * m["heads"] * m["vdim"], 0.0)),
        "mixer_out": mix(lambda m, layer: _product(n, W, m["heads"] * m["vdim"])),
        "moe_ids": mlp(lambda f, layer: (4.0 * f["router"]["experts"] * W + 2.0 * n * W, 0.0)),
        "moe_sorted": mlp(lambda f, layer: (12.0 * n * f["router"]["top"], 0.0)),
        "moe_rows": mlp(lambda f, layer: (4.0 * n * f["router"]["top"] * W, 0.0)),
        # (gate/up product with act(gate) * up in its epilogue)
        "moe_act": mlp(lambda f, layer: (2.0 * (touched(f) * 2 * f["expert"]["ff"] * W + n * f["router"]["top"] * (W + f["expert"]["ff"])),
                                         2.0 * n * f["router"]["top"] * 2 * f["expert"]["ff"] * W)),
        "moe_expert_out": mlp(lambda f, layer: (2.0 * (touched(f) * f["expert"]["ff"] * W + n * f["router"]["top"] * (W + f["expert"]["ff"])),
                                                2.0 * n * f["router"]["top"] * f["expert"]["ff"] * W)),
        # (a routed layer's shared expert ends at the same taps as a dense feed-forward: its sizes are taken then)
        "ffn_act": mlp(lambda f, layer: _product(n, 2 * (f["ff"] if f["kind"] == "dense" else f["shared"]["ff"]), W)),
        "moe_shared_out": mlp(lambda f, layer: _product(n, W, f["shared"]["ff"])),
        "ffn_out": mlp(lambda f, layer: _product(n, W, f["ff"]) if f["kind"] == "dense" else (2.0 * n * W * (f["router"]["top"] + 2), 0.0)),
    }


RESOLORN_PHASES = {"norm1": "add + norm", "latent_down": "down products (query latent, latent, gates)", "latent_q": "latent norms + cache write",
                   "q_heads": "query up product", "q_latent": "queries into the latent's space (a product a head)",
                   "attn_out": "attention over latents", "attn_values": "values out of the latent's space (a product a head)",
                   "attn_heads": "head gates", "mixer_out": "output product", "moe_ids": "router", "moe_sorted": "grouping by expert",
                   "moe_rows": "rows into the experts' order", "moe_act": "experts' gate/up products + activation",
                   "moe_expert_out": "experts' down products",
                   "ffn_act": "gate/up product + activation", "moe_shared_out": "down product", "ffn_out": None}


def qwen3_costs(raw, starts, counts):
    n, h, inter = sum(counts), raw["hidden_size"], raw["intermediate_size"]
    nq, nkv, hd = raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"]
    cached = sum(s + c for s, c in zip(starts, counts))
    return {
        "norm1": lambda layer: (n * h * 12.0, 0.0), "norm2": lambda layer: (n * h * 12.0, 0.0),
        "qkv": lambda layer: _product(n, (nq + 2 * nkv) * hd, h),
        "q_rot": lambda layer: (4.0 * n * (nq + 2 * nkv) * hd, 0.0),
        "attn_out": lambda layer: (4.0 * cached * nkv * hd + 4.0 * n * nq * hd, 4.0 * _keys_seen(starts, counts, 0) * nq * hd),
        "mixer_out": lambda layer: _product(n, h, nq * hd),
        "ffn_act": lambda layer: _product(n, 2 * inter, h),
        "ffn_out": lambda layer: _product(n, h, inter),
    }


QWEN3_PHASES = {"norm1": "add + norm", "norm2": "add + norm", "qkv": "q/k/v product", "q_rot": "norm + rotation + cache write",
                "attn_out": "attention", "mixer_out": "output product", "ffn_act": "gate/up product + activation", "ffn_out": "down product"}


def phase_table(engine, seqs, costs, names, layer_of, pk, reps, warmup):
    """One forward pass over ``seqs`` captured with an event at every named tap, replayed ``reps`` times: rows of
    (phase, calls, mean us, bytes, flops, fraction of its roofline), kernels in the order they run."""
    import torch
    from rust_mlx_b200.engine.batch import build_batch
    e = engine
    batch = build_batch(seqs, e.pools, e.device, e._status, e.vocab_size)
    marks = []

    def tap(name, tensor):
        ev = torch.cuda.Event(enable_timing=True, external=True)
        ev.record()
        marks.append((name, getattr(e, "_run_index", 0), ev))

    def step():
        marks.clear()
        tap("start", None)
        tap("nothing", None)
        e.forward(batch)
    e.forward(batch)
    torch.cuda.synchronize()
    e._ctx.tap = tap
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
    finally:
        e._ctx.tap = None
    sums = {}
    order = []
    event_us = 0.0
    for _ in range(warmup):
        graph.replay()
    for _ in range(reps):
        graph.replay()
        torch.cuda.synchronize()
        last = marks[0][2]
        for name, run, ev in marks[1:]:
            if name == "nothing":
                event_us += last.elapsed_time(ev) * 1e3
                last = ev
                continue
            if name == "ffn_out" and names.get(name, name) is None:
                # (the routed layer's last tap is its weighted sum; a dense layer's is its down product)
                label = "weighted sum of the experts" if (layer_of(run).get("mlp") or {}).get("kind") == "moe" else "down product"
            elif name not in names or name not in costs:
                continue
            else:
                label = names[name]
            layer = layer_of(run)
            if callable(label):     # (a tap that two kinds of layer share)
                label = label(layer)
            cost = costs[name](layer)
            if cost is None:
                continue
            b, f = cost
            key = label
            if key not in sums:
                sums[key] = [0.0, 0, 0.0, 0.0]
                order.append(key)
            sums[key][0] += last.elapsed_time(ev) * 1e3
            sums[key][1] += 1
            sums[key][2] += b
            sums[key][3] += f
            last = ev
    event_us /= reps
    rows = []
    for key in order:
        us_total, calls, b, f = sums[key]
        us = max(us_total / calls - event_us, 0.01)
        b, f = b / calls, f / calls
        floor_us = max(b / (pk["hbm_gbs"] * 1e3), f / (pk["bf16_tflops"] * 1e6))
        rows.append({"phase": key, "calls_per_step": calls // reps, "us": round(us, 2), "mbytes": round(b / 1e6, 3), "gflop": round(f / 1e9, 3),
                     "bound": "hbm" if b / (pk["hbm_gbs"] * 1e3) >= f / (pk["bf16_tflops"] * 1e6) else "tensor", "frac": round(floor_us / us, 4)})
    return rows, event_us


def family_bench(a):
    """Decode (batch ``a.batch`` at context CONTEXT) and prefill (PREFILL_TOKENS tokens) of Resolorn layers beside Qwen3
    layers of equal width, depth, head size and feed-forward width, with every phase against its roofline."""
    import torch
    from rust_mlx_b200.config import GugalornConfig, Qwen3Config, ResolornConfig, ReveraxConfig, SosuvikConfig
    from rust_mlx_b200.engine import Engine
    from rust_mlx_b200.engine.batch import SequenceInput
    pk = peaks()
    gug, sos, rev = a.family == "gugalorn", a.family == "sosuvik", a.family == "reverax"
    sizes = GUGALORN_SIZES if gug else SOSUVIK_SIZES if sos else REVERAX_SIZES if rev else FAMILY_SIZES
    out = {"metric": f"{a.family.capitalize()} beside {'Resolorn and ' if sos else 'Gugalorn and ' if rev else ''}Qwen3 at equal layer sizes: decode and prefill tok/s, phases against their rooflines", "impl": "ours",
           "dtype": "bf16", "data": "synthetic", "n_gpus": 1, "batch": a.batch, "context": CONTEXT, "prefill_tokens": PREFILL_TOKENS,
           "peaks": pk, "sizes": {}}
    for size in (a.family_size.split(",") if a.family_size else sorted(sizes)):
        s = sizes[size]
        groups = max(1, a.family_layers // 4)
        same = FAMILY_SIZES[size] if sos else s        # (the Resolorn layers of the same name have the sizes Sosuvik lacks)
        raw_r = gugalorn_shape(groups=groups, **s) if gug else sosuvik_shape(groups=groups, **s) if sos else \
            reverax_shape(groups=groups, **s) if rev else resolorn_shape(groups=groups, **s)
        raw_q = dict(QWEN3_8B, num_hidden_layers=4 * groups, hidden_size=s["width"], num_attention_heads=s["heads"],
                     num_key_value_heads=s["kv_heads"] if gug or sos or rev else max(1, s["heads"] // 4), head_dim=s["dim"],
                     intermediate_size=same["ff"], vocab_size=s["vocab"], max_position_embeddings=2 * MAX_CONTEXT)
        result = {}
        mine = ("gugalorn", raw_r, GugalornConfig.from_dict(raw_r), gugalorn_costs, GUGALORN_PHASES) if gug else \
               ("sosuvik", raw_r, SosuvikConfig.from_dict(raw_r), sosuvik_costs, SOSUVIK_PHASES) if sos else \
               ("reverax", raw_r, ReveraxConfig.from_dict(raw_r), reverax_costs, REVERAX_PHASES) if rev else \
               ("resolorn", raw_r, ResolornConfig.from_dict(raw_r), resolorn_costs, RESOLORN_PHASES)
        others = []
        if sos:
            raw_o = resolorn_shape(groups=groups, **same)
            others.append(("resolorn", raw_o, ResolornConfig.from_dict(raw_o), resolorn_costs, RESOLORN_PHASES))
        if rev:
            raw_o = gugalorn_shape(groups=groups, **GUGALORN_SIZES[size])
            others.append(("gugalorn", raw_o, GugalornConfig.from_dict(raw_o), gugalorn_costs, GUGALORN_PHASES))
        others.append(("qwen3", raw_q, Qwen3Config.from_dict(raw_q), qwen3_costs, QWEN3_PHASES))
        for family, raw, cfg, costs_of, names in (mine, *others):
            cache_tokens = a.batch * (CONTEXT + 2 * PAGE + a.steps + a.warmup + 64) + 2 * PREFILL_TOKENS
            engine = Engine(cfg, dtype="bfloat16", random_weights=True, seed=0, max_tokens=cache_tokens, page_size=PAGE,
                            max_requests=a.batch + 4, tuning=a.policy)
            for grp in engine.pools.paged_groups:
                grp.k_pool.normal_(0, 1)
                if grp.v_pool is not None:
                    grp.v_pool.normal_(0, 1)
            ms, launches, clock_info = time_decode(engine, a.batch, a.steps, a.warmup, ClockSampler())
            pf_ms = time_prefill(engine, PREFILL_TOKENS)
            if family == "qwen3":
                layer_of = lambda run: {}
            elif family == "reverax":       # (every layer of the configuration is a run, also one that uses another's tensors)
                layer_of = lambda run, raw=raw: raw["layers"][run]
            else:       # a run of the schedule is a layer, or (past the layers) a loop's entry
                layer_of = lambda run, raw=raw, calls=engine._calls: (raw["layers"][calls[run][0].layer]
                                                                      if calls[run][0].layer < len(raw["layers"]) else {"type": "loop"})
            # phases of a decode step and of a prompt
            run = DecodeRun(engine, a.batch, CONTEXT)
            try:
                for r in run.rids:
                    engine.pools.table.reserve(r, run.len + 1)
                seqs = [SequenceInput(r, run.len, [run.ids[0][i]], [0]) for i, r in enumerate(run.rids)]
                decode_rows, ev_us = phase_table(engine, seqs, costs_of(raw, [CONTEXT] * a.batch, [1] * a.batch), names, layer_of, pk,
                                                 max(10, a.steps // 10), a.warmup)
            finally:
                run.close()
            rid = 30_000
            engine.pools.open(rid)
            engine.pools.table.reserve(rid, PREFILL_TOKENS)
            try:
                g = torch.Generator().manual_seed(2)
                ids = torch.randint(0, engine.vocab_size, (PREFILL_TOKENS,), generator=g).tolist()
                prefill_rows, _ = phase_table(engine, [SequenceInput(rid, 0, ids, [PREFILL_TOKENS - 1])],
                                              costs_of(raw, [0], [PREFILL_TOKENS]), names, layer_of, pk, 5, 2)
            finally:
                engine.pools.table.close(rid)
            engine.check_status()
            result[family] = {"decode_tok_per_s": round(a.batch * 1000.0 / ms, 1), "decode_ms_per_step": round(ms, 4),
                              "prefill_tok_per_s": round(PREFILL_TOKENS / (pf_ms * 1e-3), 1), "prefill_ms": round(pf_ms, 3),
                              "layers": 4 * groups, "launches_per_decode_step": launches // a.steps, "clocks": clock_info,
                              "decode_phases": decode_rows, "prefill_phases": prefill_rows, "event_us": round(ev_us, 2)}
            for mode, rows in (("decode", decode_rows), ("prefill", prefill_rows)):
                print(f"-- {family} {size} {mode}: {result[family][mode + '_tok_per_s' if mode == 'decode' else 'prefill_tok_per_s']} tok/s", file=sys.stderr)
                for r_ in rows:
                    print(f"  {r_['phase']:52s} x{r_['calls_per_step']:<3d} {r_['us']:10.2f} us {r_['mbytes']:10.2f} MB {r_['gflop']:10.2f} GF "
                          f"{r_['bound']:7s} {r_['frac']:7.3f}", file=sys.stderr)
            del engine
            torch.cuda.empty_cache()
        out["sizes"][size] = {"shape": s, **result}
    print(json.dumps(out))
    return 0


def main():
    global CONTEXT, MAX_CONTEXT
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=QWEN3_8B["num_hidden_layers"])
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 / 64, prefill and e2e")
    ap.add_argument("--prefill-only", action="store_true", help="time the 2,048-token prefill only (for profiling it)")
    ap.add_argument("--portion-at", type=int, default=0, metavar="CONTEXT",
                    help="instead: time one 512-token portion of a prompt whose first CONTEXT tokens are in the cache (chunked "
                         "prefill of a long prompt); prints its own JSON line")
    ap.add_argument("--per-kernel", action="store_true",
                    help="instead: time the phases of one decode step one by one and print each one's bytes, time and "
                         "fraction of the memory peak")
    ap.add_argument("--shape", default="qwen3-8b", choices=sorted(SHAPES), help="layer sizes (default: the Qwen3-8B shape)")
    ap.add_argument("--context", type=int, default=CONTEXT, help="tokens each request holds when decoding starts")
    ap.add_argument("--continuous", action="store_true",
                    help="instead: 64 requests with prompts of 128..3072 random ids, 256 tokens each, through the "
                         "scheduler with chunked prefill of 512 (continuous batching); prints its own JSON line")
    ap.add_argument("--family", default="", choices=["", "resolorn", "gugalorn", "sosuvik", "reverax"],
                    help="instead: layers of this design at sizes of real models beside Qwen3 layers of equal width, depth, head "
                         "size and feed-forward width: decode and prefill tok/s and every phase against its roofline; prints its own "
                         "JSON line")
    ap.add_argument("--family-size", default="", help="with --family: which sizes, comma separated (default: all of " + ", ".join(sorted(FAMILY_SIZES)) + ")")
    ap.add_argument("--family-layers", type=int, default=4, help="with --family: layers (a multiple of four)")
    ap.add_argument("--policy", default="auto", choices=["auto", "measured", "all", "none"],
                    help="which products of few rows take the tcgen05 kernel (auto: time both when the engine starts)")
    a = ap.parse_args()
    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust/MLX/Metal program for Apple GPUs: no Rust toolchain, no MLX and no "
                          "setup.py/pyproject.toml here (pip: 'not installable'), so it cannot be built or run on this box"}))
        return 0
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    a.warmup = max(a.warmup, 3)

    import torch
    from rust_mlx_b200.config import Qwen3Config
    from rust_mlx_b200.engine import Engine

    CONTEXT = a.context
    if a.family:
        MAX_CONTEXT = max(MAX_CONTEXT, 2 * CONTEXT)
        return family_bench(a)
    base = SHAPES[a.shape]
    if a.shape != "qwen3-8b" and a.layers == QWEN3_8B["num_hidden_layers"]:
        a.layers = base["num_hidden_layers"]
    MAX_CONTEXT = max(MAX_CONTEXT, 2 * CONTEXT)
    raw = dict(base, num_hidden_layers=a.layers, max_position_embeddings=MAX_CONTEXT)
    cfg = Qwen3Config.from_dict(raw)
    if a.continuous:
        return continuous(cfg, raw, a)
    if a.portion_at:
        CONTEXT = a.portion_at
    biggest = 1 if (a.no_points or a.prefill_only or a.per_kernel or a.portion_at) else max(64, a.batch)
    cache_tokens = max(biggest, a.batch) * (CONTEXT + 2 * PAGE + a.steps + a.warmup + 64)
    engine = Engine(cfg, dtype="bfloat16", random_weights=True, seed=0, max_tokens=cache_tokens, page_size=PAGE,
                    max_requests=max(biggest, a.batch) + 2, tuning=a.policy)
    for grp in engine.pools.paged_groups:      # synthetic cache contents for the requests that start at CONTEXT
        grp.k_pool.normal_(0, 1)
        grp.v_pool.normal_(0, 1)
    pk = peaks()
    if a.per_kernel:
        return per_kernel(engine, raw, a, pk)
    if a.portion_at:
        portion = 512
        ms = time_prefill(engine, portion, start_at=a.portion_at)
        _, per_layer, head = model_bytes(raw, a.layers)
        gemm = 2.0 * portion * a.layers * per_layer + 2.0 * head
        # every query of the portion against the cache's keys and, causally, the portion's own (half of them on average)
        attn = 4.0 * portion * (a.portion_at + portion / 2) * raw["head_dim"] * raw["num_attention_heads"] * a.layers
        print(json.dumps({"metric": f"prompt portion of {portion} tokens at context {a.portion_at} ({a.shape} shape, bf16)",
                          "value": round(portion / (ms * 1e-3), 1), "unit": "tok/s", "ms": round(ms, 3), "layers": a.layers,
                          "tflop": round((gemm + attn) / 1e12, 2), "attention_share_of_flop": round(attn / (gemm + attn), 3),
                          "frac": round((gemm + attn) / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "of": pk["source"]}))
        return 0
    if a.prefill_only:
        pf_ms = time_prefill(engine, PREFILL_TOKENS)
        flops = prefill_flops(raw, a.layers, PREFILL_TOKENS)
        print(json.dumps({"prefill": {"value": round(PREFILL_TOKENS / (pf_ms * 1e-3), 1), "tokens": PREFILL_TOKENS,
                                      "ms": round(pf_ms, 3), "layers": a.layers,
                                      "frac": round(flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}}))
        return 0

    clocks = ClockSampler()
    ms, launches, clock_info = time_decode(engine, a.batch, a.steps, a.warmup, clocks)
    value = a.batch * 1000.0 / ms
    weight_bytes, _, _ = model_bytes(raw, a.layers)
    step_bytes = weight_bytes + a.batch * (CONTEXT + a.warmup + a.steps / 2) * kv_bytes_per_token(raw, a.layers)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    line = {
        "metric": f"decode tok/s at batch {a.batch}, context {CONTEXT} ({a.shape} shape, bf16)", "value": round(value, 2), "unit": "tok/s",
        "n_gpus": 1, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": a.shape + " shape, random weights", "layers": a.layers, "layers_full": base["num_hidden_layers"],
                   "hidden": raw["hidden_size"], "q_heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
                   "head_dim": raw["head_dim"], "intermediate": raw["intermediate_size"],
                   "vocab": raw["vocab_size"], "global_batch": a.batch, "seq_len": CONTEXT, "max_context": MAX_CONTEXT,
                   "page_size": PAGE, "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU",
                   "l2": f"inputs larger than L2 ({weight_bytes / 1e9:.0f} GB of weights per step), no flush",
                   "peaks": pk["source"]},
        "gpu_launches": launches, "clocks": clock_info,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"]},
    }
    if not a.no_points:
        points = {}
        for b in (1, 64):
            pms, _, _ = time_decode(engine, b, max(8, a.steps // 2), a.warmup)
            points[f"decode_b{b}"] = round(b * 1000.0 / pms, 2)
        line["points"] = points
        pf_ms = time_prefill(engine, PREFILL_TOKENS)
        flops = prefill_flops(raw, a.layers, PREFILL_TOKENS)
        line["prefill"] = {"value": round(PREFILL_TOKENS / (pf_ms * 1e-3), 1), "tokens": PREFILL_TOKENS, "ms": round(pf_ms, 3),
                           "frac": round(flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "of": pk["source"]}
        e2e, h2d, d2h, checked = time_e2e(engine, a.batch, max(128, a.steps))
        line["e2e"] = {"value": round(e2e, 2), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
        line["checked"] = checked
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
