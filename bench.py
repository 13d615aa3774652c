#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at LFM2-1.2B sizes with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 4096] [--layers N] [--dtype bfloat16|float32]

One JSON line on stdout.  ``value`` is decoded tokens per second at the given batch, device-
timed with CUDA events over regions of exactly K decode steps (each step: the packed index data
goes host->device, the captured decode graph replays, greedy tokens are chosen on the device).
The region is repeated, each time over the same positions of the same requests, until at least
0.3 s of device time has been measured, and the median region is reported, so that a small K
still gives a steady figure.  ``e2e`` is the same metric through the engine loop a user drives
(scheduler, step, sampler, host tokens in and out, wall clock).  ``prefill`` times one
2,048-token prompt in one step; ``roofline`` relates the decode step to the bytes it must read;
``kernels`` says where the decode step's and the prefill's time goes, kernel family by kernel
family, each against the measured peak that bounds it; ``points`` holds decode at batch 1 and 64
and the true 32-bit path's figures.  Peaks come from MEASURED_PEAKS.json when the file is there,
else from the fallback figures.

The engine runs on one GPU: with --gpus above 1 it says so and exits with 2.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# LFM2-1.2B layer sizes: full_attention at layers 2, 5, 8, 10, 12, 14 of 16
LFM2_1P2B = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 65536, "hidden_size": 2048, "intermediate_size": 12288,
    "block_auto_adjust_ff_dim": True, "block_ffn_dim_multiplier": 1.0, "block_multiple_of": 256,
    "num_hidden_layers": 16, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "conv_L_cache": 3, "conv_bias": False, "rope_theta": 1000000.0, "norm_eps": 1e-5,
    "tie_word_embeddings": True, "max_position_embeddings": 128000,
    "layer_types": ["full_attention" if l in (2, 5, 8, 10, 12, 14) else "conv" for l in range(16)],
}


def lfm2_sizes(name):
    """The other two sizes the benchmark configurations name (random weights, so only the layer
    sizes matter).  The 2.6B stack has 8 attention layers among 30; they are spread evenly here."""
    cfg = dict(LFM2_1P2B)
    if name == "1.2b":
        return cfg
    if name == "700m":
        cfg.update(hidden_size=1536, intermediate_size=10240, num_attention_heads=24)
        return cfg
    if name == "2.6b":
        attn = (2, 6, 10, 14, 18, 21, 24, 27)
        cfg.update(intermediate_size=10752, num_hidden_layers=30,
                   layer_types=["full_attention" if l in attn else "conv" for l in range(30)])
        return cfg
    raise ValueError(name)


def peaks():
    p = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                m = json.load(f)
            for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                if isinstance(m.get(k), (int, float)):
                    p[k] = float(m[k])
            p["source"] = "measured"
        except (OSError, ValueError):
            pass
    return p


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm = sorted(int(r[0]) for r in self.rows if len(r) >= 6 and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) >= 6 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def part_tensors(plan):
    """(label, tensor) for every tensor that a part of the plan holds, each tensor once; the label is
    the part's class and attribute name, e.g. ``SwiGLU.w_gate_up``.  Walks whatever parts the
    blocks are made of, so a plan of other parts needs no change here."""
    import torch
    from vapi_b200.parts.base import Part
    seen = set()

    def of_part(part):
        for name, v in vars(part).items():
            if isinstance(v, torch.Tensor) and v.data_ptr() not in seen:
                seen.add(v.data_ptr())
                yield f"{type(part).__name__}.{name}", v
        for v in vars(part).values():
            if isinstance(v, Part):
                yield from of_part(v)

    for call in plan.order:
        yield from of_part(plan.layers[call.layer])
    yield from of_part(plan.final_norm)
    yield from of_part(plan.head)        # tied: the embedding table, read once by the head
    yield from of_part(plan.embedding)


def model_numbers(runner):
    """Bytes of every weight a decode step reads once (the embedding table counts once: a step
    gathers a few rows of it and the tied head reads all of it), and matrix-product parameters."""
    wbytes, mm_params = 0, 0
    for label, t in part_tensors(runner.plan):
        if label == "TokenEmbedding.table":
            continue                      # (reached only when untied) a table is gathered from, not streamed
        wbytes += t.numel() * t.element_size()
        if t.dim() == 2 and t.shape[0] > 8:
            mm_params += t.numel()
    return wbytes, mm_params


def trace_table(events):
    """Rows for the last whole step among the stamps: the step's kernels in the order in which their
    dependency waits returned, each with how long it then took until the next kernel's wait returned
    (its own dependent work, its drain and the hand-over)."""
    rel = [e for e in events if e["kind"] == "released"]
    ends = [i for i, e in enumerate(rel) if e["library"] == "sampling"]
    if len(ends) < 2:
        return []
    step = rel[ends[-2] + 1:ends[-1] + 1]
    start = {}
    for e in events:
        if e["kind"] == "start":
            start.setdefault((e["library"], e["blocks"], e["threads"]), []).append(e["ns"])
    rows = []
    for a, b in zip(step, step[1:] + [None]):
        key = (a["library"], a["blocks"], a["threads"])
        began = max((t for t in start.get(key, []) if t <= a["ns"]), default=a["ns"])
        rows.append({"library": a["library"], "blocks": a["blocks"], "threads": a["threads"],
                     "waited_us": (a["ns"] - began) / 1e3, "at_us": (a["ns"] - step[0]["ns"]) / 1e3,
                     "until_next_us": (b["ns"] - a["ns"]) / 1e3 if b else None})
    return rows


#: the calls that are matrix products (time against the tensor peak); the rest move bytes
PRODUCTS = ("linear", "skinny_linear", "linear_tc", "prompt_linear", "skinny_shortconv")

#: the package's kernels as the parts call them, with the library each lives in
OPS = {"embed": "elementwise", "add_residual_ss": "elementwise", "resolve_tokens": "elementwise",
       "add_rmsnorm": "elementwise", "add_residual": "elementwise", "swiglu": "elementwise",
       "skinny_linear": "gemv", "skinny_shortconv": "gemv", "linear_tc": "linear_tc", "prompt_linear": "linear_prompt",
       "rope_cos_sin": "rope",
       "qk_norm_rope_write": "rope", "paged_attention": "attention", "decode_attention_fused": "attention",
       "shortconv": "shortconv", "sample_rows": "sampling", "sample_truncated": "sampling", "linear": "library"}


class OpLog:
    """Stands between the parts and the kernels' Python faces for one measurement: every call is
    noted with the weight it streams (the first 2-D bfloat16/float32 matrix among its arguments
    that a part of the plan holds), the kernels it launched and, when ``events`` is set, CUDA
    events around it.  Calls made from inside another noted call are not noted again."""

    def __init__(self, ops, plan, events=False):
        import torch
        self.ops, self.torch, self.events = ops, torch, events
        self.labels = {t.data_ptr(): (label, t) for label, t in part_tensors(plan)}
        self.calls, self.depth, self.saved = [], 0, {}

    def __enter__(self):
        for name in OPS:
            fn = getattr(self.ops, name)
            self.saved[name] = fn
            setattr(self.ops, name, self._wrap(name, fn))
        return self

    def __exit__(self, *exc):
        for name, fn in self.saved.items():
            setattr(self.ops, name, fn)

    def _wrap(self, name, fn):
        torch = self.torch

        def call(*a, **kw):
            if self.depth:
                return fn(*a, **kw)
            self.depth += 1
            try:
                tensors = [t for t in list(a) + list(kw.values()) if isinstance(t, torch.Tensor)]
                weight = next((self.labels[t.data_ptr()] for t in tensors if t.data_ptr() in self.labels and t.dim() == 2), None)
                before = self.ops.launch_count
                ev = None
                if self.events:
                    ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                    ev[0].record()
                out = fn(*a, **kw)
                if ev:
                    ev[1].record()
                outs = [t for t in (out if isinstance(out, tuple) else (out,)) if isinstance(t, torch.Tensor)]
                rows = max([t.shape[0] for t in outs if t.dim() >= 1] or [0])
                # what an elementwise call moves: its activations in and out (not the caches and states it
                # touches a few rows of, not the plan's own tensors)
                moved = sum(t.numel() * t.element_size() for t in tensors + outs
                            if t.dim() <= 2 and t.data_ptr() not in self.labels)
                if name == "embed":
                    moved *= 2            # the rows gathered from the table, and the stream written
                self.calls.append({"op": name, "weight": weight[0] if weight else None,
                                   "weight_shape": tuple(weight[1].shape) if weight else None,
                                   "weight_bytes": weight[1].numel() * weight[1].element_size() if weight else 0,
                                   "rows": rows, "moved_bytes": moved, "launches": self.ops.launch_count - before, "events": ev})
                return out
            finally:
                self.depth -= 1
        return call


def family_of(call):
    """The name under which a noted call is summed up: a product by the matrix it streams, any
    other kernel by its own name."""
    if call["op"] in PRODUCTS and call["weight"]:
        return call["weight"] + ("+conv" if call["op"] == "skinny_shortconv" else "")
    return call["op"]


def decode_kernel_table(args, pk, timeout=420):
    """Where the captured decode step's time goes: a second process runs a few steps of the same
    step with a measuring build of every kernel library (its kernels stamp the device clock) and
    names the kernels in launch order; this sums them up by family.  Each family's time is the time
    from the return of its kernels' dependency waits to the return of the next kernel's, so the
    families add up to the step; bytes are the weights and cache it has to read."""
    cmd = [sys.executable, os.path.abspath(__file__), "--only", "trace", "--rows-json", "--steps", "6", "--warmup", "4",
           "--batch", str(args.batch), "--context", str(args.context), "--sizes", args.sizes, "--layers", str(args.layers),
           "--page-size", str(args.page_size)]
    try:
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)
        line = next((l for l in proc.stdout.splitlines() if l.startswith('{"trace_rows"')), None)
        if proc.returncode != 0 or line is None:
            return {"unavailable": "the measuring pass failed: " + (proc.stderr.strip().splitlines() or ["no output"])[-1][:200]}
        rec = json.loads(line)
    except (subprocess.TimeoutExpired, OSError, ValueError) as e:
        return {"unavailable": f"the measuring pass failed: {type(e).__name__}"}
    if rec.get("mismatch"):
        return {"unavailable": rec["mismatch"]}
    fam = {}
    for r in rec["trace_rows"]:
        f = fam.setdefault(r["family"], {"us": 0.0, "bytes": 0, "launches": 0})
        f["us"] += r["us"] or 0.0
        f["bytes"] += r["bytes"]
        f["launches"] += 1
    out = {}
    for name, f in sorted(fam.items(), key=lambda kv: -kv[1]["us"]):
        gbs = f["bytes"] / (f["us"] * 1e-6) / 1e9 if f["us"] > 0 else 0.0
        out[name] = {"us": round(f["us"], 1), "launches": f["launches"], "MB": round(f["bytes"] / 1e6, 1),
                     "GBps": round(gbs, 0), "frac_hbm": round(gbs / pk["hbm_gbs"], 3)}
    return {"ms_per_step_with_stamps": rec["ms_per_step"], "families": out}


def run(args):
    if args.only == "trace":          # a measuring build of every kernel library, named before the first import
        os.environ["VAPI_NVCC_FLAGS"] = (os.environ.get("VAPI_NVCC_FLAGS", "") + " -DVAPI_TRACE").strip()
    import torch
    from vapi_b200 import ops
    from vapi_b200.engine.engine import Engine
    from vapi_b200.engine.runner import ModelRunner, parse_dtype
    from vapi_b200.engine.scheduler import SchedulerConfig
    from vapi_b200.engine.step import StepEntry
    from vapi_b200.sampling.params import SamplingParams

    pk = peaks()
    cfg = lfm2_sizes(args.sizes)
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    if args.only == "serve":
        return serve(args, cfg)
    if layers != full_layers:
        cfg["num_hidden_layers"] = layers
        cfg["layer_types"] = cfg["layer_types"][:layers]
    ctx_len, B = args.context, args.batch
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    max_b = max(B, 64)
    page = args.page_size or ModelRunner.default_page_size
    gen = torch.Generator().manual_seed(1)
    vocab = cfg["vocab_size"]
    MIN_TIMED_S = 0.3

    def make_runner(dtype, most_requests=max_b):
        n_pages = most_requests * (-(-(ctx_len + 256) // page)) + 8      # (the engine-loop run lets contexts grow past ctx_len)
        return ModelRunner.from_random(cfg, seed=0, dtype=dtype, device="cuda:0", num_pages=n_pages, page_size=page,
                                       max_requests=most_requests, max_batched_tokens=8192, max_context=ctx_len + 256,
                                       watermark=0.0, validate=False)

    def fill(runner, batch, length):
        """Open `batch` requests and prefill them to `length` tokens in portions (untimed)."""
        rcs = []
        for i in range(batch):
            rc = runner.cache.open(("bench", batch, i))
            toks = torch.randint(0, vocab, (length,), generator=gen).tolist()
            pos = 0
            while pos < length:
                q = min(4096, length - pos)
                assert runner.cache.reserve(rc, pos + q)
                runner.step([StepEntry(rc, toks[pos:pos + q], [])])
                pos += q
            rcs.append(rc)
        torch.cuda.synchronize()
        return rcs

    def decode_steps(runner, rcs, count, timed):
        """`count` decode steps on the stream; device time in ms when `timed`."""
        toks = torch.randint(0, vocab, (count, len(rcs)), generator=gen).tolist()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for s in range(count):
            entries = []
            for j, rc in enumerate(rcs):
                assert runner.cache.reserve(rc, rc.num_tokens + 1)
                entries.append(StepEntry(rc, [toks[s][j]], [0]))
            logits = runner.step_decode_graph(entries)
            if logits is None:
                logits = runner.step(entries)
            ops.sample_rows(logits)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) if timed else 0.0

    def decode_point(runner, batch, steps, warmup, clocks=None, min_s=MIN_TIMED_S):
        """Regions of exactly `steps` decode steps that end at the context length, repeated until
        `min_s` seconds of device time are measured (three regions at least); every region decodes
        the same positions of the same requests again (the requests' counts of computed positions
        are set back in between, which leaves their pages in place).  Returns the median region."""
        start_len = ctx_len - steps - 1
        rcs = fill(runner, batch, start_len)

        def rewind():
            for rc in rcs:
                runner.cache.commit(rc, start_len)

        done = 0
        while done < warmup:
            k = min(steps, warmup - done)
            decode_steps(runner, rcs, k, False)
            rewind()
            done += k
        if clocks:
            clocks.start()
        regions, total, launches = [], 0.0, 0
        while len(regions) < 3 or (total < min_s * 1e3 and len(regions) < 400):
            before = ops.launch_count
            ms = decode_steps(runner, rcs, steps, True)
            launches = ops.launch_count - before
            kv_bytes = sum(rc.num_tokens for rc in rcs) * runner.cache.bytes_per_token() + \
                batch * runner.cache.state_bytes_per_request()
            rewind()
            regions.append(ms)
            total += ms
        clk = clocks.stop() if clocks else None
        for rc in rcs:
            runner.cache.close(rc)
        ms = sorted(regions)[len(regions) // 2]
        return ms, launches, clk, kv_bytes, len(regions)

    if args.only == "trace":
        return trace_pass(args, make_runner(args.dtype), fill, decode_steps, ops, ctx_len, B)
    dtype = "float32" if parse_dtype(args.dtype) == torch.float32 else "bfloat16"
    runner = make_runner(dtype)
    wbytes, mm_params = model_numbers(runner)
    fp32_peak = measure_fp32_peak(dev) if (dtype == "float32" or args.only == "all") else None
    peak_tflops = fp32_peak if dtype == "float32" else pk["bf16_tflops"]
    if args.only == "prefill":
        p, fam = measure_prefill(runner, ops, mm_params, pk, peak_tflops, gen, vocab, dev, warm=max(1, min(args.warmup, 3)),
                                 iters=max(1, min(args.steps, 5)))
        print(json.dumps({"only": "prefill", "dtype": dtype, "prefill": p, "kernels": fam}), flush=True)
        return 0
    # ---- headline: decode at the given batch -----------------------------------------
    clocks = ClockSampler()
    ms, launches, clk, kv_bytes, regions = decode_point(runner, B, args.steps, args.warmup, clocks)
    ms_step = ms / args.steps
    value = B * args.steps / (ms / 1e3)
    print(f"[bench] decode b{B} {dtype}: {value:.0f} tok/s, {ms_step:.4f} ms/step (median of {regions} regions of "
          f"{args.steps} steps)", file=sys.stderr, flush=True)
    step_bytes = wbytes + kv_bytes
    achieved = step_bytes / (ms_step / 1e3) / 1e9

    if args.only == "decode":
        print(json.dumps({"only": "decode", "dtype": dtype, "value": round(value, 1), "ms_per_step": round(ms_step, 4),
                          "gpu_launches": launches, "roofline_frac": round(achieved / pk["hbm_gbs"], 4)}), flush=True)
        return 0
    # ---- other batch sizes ----------------------------------------------------------
    points = {}
    for b in (1, 64):
        m, _, _, kvb, _ = decode_point(runner, b, args.steps, max(8, args.warmup))
        points[f"decode_b{b}"] = round(b * args.steps / (m / 1e3), 1)
        points[f"decode_b{b}_frac_hbm"] = round((wbytes + kvb) / (m / args.steps / 1e3) / 1e9 / pk["hbm_gbs"], 4)
        print(f"[bench] decode b{b} {dtype}: {points[f'decode_b{b}']} tok/s, {m / args.steps:.4f} ms/step, "
              f"{points[f'decode_b{b}_frac_hbm']} of the HBM peak", file=sys.stderr, flush=True)

    prefill, prefill_families = measure_prefill(runner, ops, mm_params, pk, peak_tflops, gen, vocab, dev)
    c = runner.plan.config
    n_attn = len(runner.cache.paged[0].sites) if runner.cache.paged else 0

    # ---- end to end through the engine loop ----------------------------------------
    # regions of `steps` engine steps, one after the other (the contexts grow): as many as 0.3 s needs, and no
    # more than keep every request below the context limit with the middle region near the context length
    warm_e2e = max(8, args.warmup)
    reps = max(1, min(int(MIN_TIMED_S * 1e3 / max(ms, 1e-3)) + 1, (512 + args.steps - 40 - warm_e2e) // args.steps))
    eng = Engine(runner, SchedulerConfig(max_concurrent_seqs=max_b, max_batched_tokens=8192,
                                         prefill_chunk_tokens=4096, max_context=ctx_len + 256), use_graphs=True)
    # the middle region ends near the context length; requests finish their prompts at different
    # steps, so leave room for the early ones
    start_len = max(16, ctx_len - warm_e2e - (reps * args.steps) // 2 - args.steps // 2 - 2)
    for i in range(B):
        prompt = torch.randint(0, vocab, (start_len,), generator=gen).tolist()
        eng.admit(("e2e", i), prompt, SamplingParams(temperature=0.0, max_tokens=warm_e2e + reps * args.steps + 128,
                                                     ignore_eos=True))
    while any(s.needs_prefill() for s in eng.scheduler.seqs.values()) or eng.scheduler.num_waiting:
        eng.step()
    for _ in range(warm_e2e):
        eng.step()
    torch.cuda.synchronize()
    st0 = dict(eng.stats.__dict__)
    e2e_regions, h2d, d2h = [], 0, 0
    for _ in range(reps):
        t0 = time.perf_counter()
        got = 0
        for _ in range(args.steps):
            out = eng.step()        # (the engine runs one step ahead: these are the tokens of the step before)
            got += len(out.new_tokens)
            h2d += runner.packer.h2d_bytes_last + eng.sampler.h2d_bytes_last
            d2h += eng.sampler.d2h_bytes_last
        torch.cuda.synchronize()
        e2e_regions.append(time.perf_counter() - t0)
        assert got == B * args.steps, (got, eng.stats, eng.last_error)
    e2e_s = sorted(e2e_regions)[len(e2e_regions) // 2]
    e2e = {"value": round(B * args.steps / e2e_s, 1), "unit": "tokens/s",
           "h2d_bytes_per_step": h2d // (reps * args.steps), "d2h_bytes_per_step": d2h // (reps * args.steps),
           "ms_per_step": round(e2e_s * 1e3 / args.steps, 4), "regions": reps}
    runner.check_status()
    st, n = eng.stats, reps * args.steps
    host = {k: round((getattr(st, k) - st0[k]) / n, 4) for k in ("schedule_ms", "forward_ms", "sample_ms", "commit_ms")}
    e2e["host_ms_per_decode_step"] = host
    print(f"[bench] e2e: {e2e}", file=sys.stderr, flush=True)
    for seq in list(eng.scheduler.seqs.values()):
        eng.cancel(seq.seq_id)
    eng.run()

    # ---- the true 32-bit path (the default run is bfloat16) -----------------------------
    if dtype == "bfloat16" and args.only == "all" and not args.no_fp32:
        del eng, runner
        torch.cuda.empty_cache()
        r32 = make_runner("float32", most_requests=max(B, 8))
        w32, mm32 = model_numbers(r32)
        for b in sorted({1, B}):
            m, _, _, kvb, _ = decode_point(r32, b, args.steps, max(8, args.warmup))
            points[f"decode_b{b}_fp32"] = round(b * args.steps / (m / 1e3), 1)
            points[f"decode_b{b}_fp32_frac_hbm"] = round((w32 + kvb) / (m / args.steps / 1e3) / 1e9 / pk["hbm_gbs"], 4)
        p32, _ = measure_prefill(r32, ops, mm32, pk, fp32_peak, gen, vocab, dev, warm=2, iters=3, families=False)
        points["prefill_fp32"] = p32["value"]
        points["prefill_fp32_ms"] = p32["ms"]
        points["prefill_fp32_frac"] = p32["frac"]
        print(f"[bench] float32: {({k: v for k, v in points.items() if 'fp32' in k})}", file=sys.stderr, flush=True)
        del r32
        torch.cuda.empty_cache()

    kernels = {"prefill": prefill_families}
    if dtype == "bfloat16" and not args.no_kernels:
        kernels[f"decode_b{B}"] = decode_kernel_table(args, pk)

    line = {
        "metric": "LFM2-%s decode tokens/s (batch %d, context %d), random weights" % (args.sizes.upper(), B, ctx_len),
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if dtype == "bfloat16" else "fp32",
        "data": "synthetic (seeded uniform-random token ids, random-init weights N(0, 0.02))",
        "impl": "vapi_b200",
        "config": {
            "model": "LFM2-%s sizes" % args.sizes.upper(), "global_batch": B, "seq_len": ctx_len, "parallelism": "single GPU",
            "layers": layers, "layers_of_configuration": full_layers, "attention_layers": n_attn,
            "hidden_size": c.hidden_size, "intermediate_size": c.intermediate_size, "vocab_size": c.vocab_size,
            "heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads, "head_dim": c.head_dim,
            "conv_L_cache": c.conv_L_cache, "page_size": page, "cuda_graphs": True,
            "l2": "inputs larger than L2 (weights %.2f GB per step)" % (wbytes / 1e9),
            "peaks": pk["source"],
            "timing": "median of %d regions of %d steps over the same positions" % (regions, args.steps),
            "fp32_peak_tflops": fp32_peak,
        },
        "e2e": e2e,
        "gpu_launches": launches,
        "clocks": clk,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes)},
        "points": points,
        "kernels": kernels,
    }
    print(json.dumps(line), flush=True)
    return 0


def trace_pass(args, runner, fill, decode_steps, ops, ctx_len, B):
    """A few decode steps of the measuring build: what one step's kernels did inside the captured
    graph, from their own time stamps; with --rows-json as one JSON line in which every kernel
    carries its family and the bytes it has to read."""
    import torch
    ops.trace_start()
    steps, warm = min(args.steps, 8), min(args.warmup, 4)
    rcs = fill(runner, B, ctx_len - steps - warm - 1)
    log = OpLog(ops, runner.plan)
    real_forward = runner.forward

    graph_calls = []

    def forward(ctx):               # the last forward pass before the steps is the one the graph holds
        log.calls.clear()
        out = real_forward(ctx)
        graph_calls[:] = list(log.calls)
        return out

    runner.forward = forward
    with log:
        decode_steps(runner, rcs, warm, False)
    runner.forward = real_forward
    ms = decode_steps(runner, rcs, steps, True)
    rows = trace_table(ops.trace_read())
    kv_per_site = sum(rc.num_tokens for rc in rcs) * runner.cache.bytes_per_token() / \
        max(1, sum(len(g.sites) for g in runner.cache.paged))
    state_per_site = B * runner.cache.state_bytes_per_request() / max(1, sum(len(g.sites) for g in runner.cache.state))
    if not args.rows_json:
        print(f"decode step, batch {B}, context {ctx_len}: {ms / steps:.4f} ms/step with the stamps on; one step's kernels in "
              f"the order in which their dependency waits returned", flush=True)
        print("   at us   library      blocks threads  waited us  until the next kernel's wait returns, us", flush=True)
        for r in rows:
            nxt = f"{r['until_next_us']:8.2f}" if r["until_next_us"] is not None else "       -"
            print(f"{r['at_us']:8.2f}   {r['library']:12s} {r['blocks']:6d} {r['threads']:7d}  {r['waited_us']:9.2f}  {nxt}", flush=True)
        return 0
    # name the stamped kernels: the graph's launches in order, then the sampler's
    expect = []
    for c in graph_calls:
        for k in range(c["launches"]):
            nbytes = (c["weight_bytes"] if c["op"] in PRODUCTS else c["moved_bytes"]) if k == 0 else 0
            if c["op"] in ("paged_attention", "decode_attention_fused") and k == 0:
                nbytes = int(kv_per_site)
            if c["op"] == "skinny_shortconv" and k == 0:
                nbytes += int(state_per_site)
            expect.append({"library": OPS[c["op"]], "family": family_of(c), "bytes": nbytes})
    expect.append({"library": "sampling", "family": "sample_rows", "bytes": B * runner.vocab_size * 4})
    out, mismatch = [], None
    if len(rows) != len(expect):
        mismatch = f"the step stamped {len(rows)} kernels where the launch log names {len(expect)}"
    else:
        for r, e in zip(rows, expect):
            if r["library"] != e["library"]:
                mismatch = f"a kernel of lib{r['library']} stands where the launch log names lib{e['library']}"
                break
            out.append({"family": e["family"], "bytes": e["bytes"], "us": r["until_next_us"], "blocks": r["blocks"]})
    print(json.dumps({"trace_rows": out, "mismatch": mismatch, "ms_per_step": round(ms / steps, 4)}), flush=True)
    return 0


def measure_fp32_peak(dev):
    """The library's float32 matrix product with every reduced-precision mode off, 4096^3, best of
    5 after 2 warm-ups, in TFLOP/s: the peak that the true 32-bit path's prefill is held against."""
    import torch
    from vapi_b200 import ops
    ops.strict_fp32()
    n = 4096
    a = torch.randn(n, n, device=dev)
    b = torch.randn(n, n, device=dev)
    best = None
    for it in range(7):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch.mm(a, b)
        e1.record()
        torch.cuda.synchronize()
        if it >= 2:
            t = e0.elapsed_time(e1)
            best = t if best is None else min(best, t)
    return round(2.0 * n ** 3 / (best / 1e3) / 1e12, 1)


def serve(args, cfg):
    """Continuous batching: --requests requests with random prompt lengths 128..2,048 arrive at
    once, each generates --max-tokens tokens (greedy); everything goes through the engine loop.
    One JSON line: generated tokens per second and all tokens (prompt + generated) per second."""
    import torch
    from vapi_b200.engine.engine import Engine
    from vapi_b200.engine.runner import ModelRunner
    from vapi_b200.engine.scheduler import SchedulerConfig
    from vapi_b200.sampling.params import SamplingParams
    R, ctx = args.requests, args.context
    page = ModelRunner.default_page_size
    runner = ModelRunner.from_random(cfg, seed=0, dtype="bfloat16", device="cuda:0",
                                     num_pages=R * (-(-(2048 + args.max_tokens + 1) // page)) + 8, max_requests=R,
                                     max_batched_tokens=8192, max_context=ctx, validate=False)
    eng = Engine(runner, SchedulerConfig(max_concurrent_seqs=R, max_batched_tokens=8192, prefill_chunk_tokens=2048,
                                         max_context=ctx))
    gen = torch.Generator().manual_seed(7)
    lens = torch.randint(128, 2049, (R,), generator=gen).tolist()

    def one_round(tag):
        for i, n in enumerate(lens):
            eng.admit((tag, i), torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist(),
                      SamplingParams(temperature=0.0, max_tokens=args.max_tokens, ignore_eos=True))
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        done = eng.run()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        assert len(done) == R and all(len(f.tokens) == args.max_tokens for f in done), eng.last_error
        return dt

    one_round("warm")           # compiles nothing new afterwards: graphs of every bucket are captured
    steps0 = eng.stats.steps
    dt = one_round("timed")
    runner.check_status()
    out_toks, in_toks = R * args.max_tokens, sum(lens)
    print(json.dumps({"only": "serve", "model": "LFM2-%s sizes" % args.sizes.upper(), "requests": R,
                      "prompt_tokens": in_toks, "generated_tokens": out_toks, "seconds": round(dt, 4),
                      "generated_tokens_per_s": round(out_toks / dt, 1),
                      "all_tokens_per_s": round((in_toks + out_toks) / dt, 1),
                      "steps": eng.stats.steps - steps0, "preemptions": eng.stats.preemptions,
                      "steps_ahead": eng.stats.ahead_steps}), flush=True)
    return 0


def measure_prefill(runner, ops, mm_params, pk, peak_tflops, gen, vocab, dev, warm=3, iters=5, families=True):
    """One 2,048-token prompt in one step, L2 flushed before each timed run; then, once more, with
    CUDA events around every kernel call of the step: where the time goes, family by family."""
    import torch
    from vapi_b200.engine.step import StepEntry
    T = 2048
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def one(tag):
        rc = runner.cache.open(("prefill", tag))
        toks = torch.randint(0, vocab, (T,), generator=gen).tolist()
        assert runner.cache.reserve(rc, T)
        flush.zero_()                                   # larger than L2: nothing of the last run stays cached
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        runner.step([StepEntry(rc, toks, [T - 1])])
        e1.record()
        torch.cuda.synchronize()
        runner.cache.close(rc)
        return e0.elapsed_time(e1)

    times = [one(it) for it in range(warm + iters)][warm:]
    pre_ms = sorted(times)[len(times) // 2]
    n_attn_sites = [s for g in runner.cache.paged for s in g.sites]
    head_params = runner.plan.head.weight.numel()
    attn_flops = 0.0
    for g in runner.cache.paged:
        # per attention call site: QK^T and PV over the causal half, 2 flops a multiply-add
        mixers = [runner.plan.layers[runner.plan.order[s].layer].mixer for s in g.sites]
        attn_flops += sum(4.0 * m.nh * m.d * (T * (T + 1) / 2) for m in mixers)
    flops = 2.0 * (mm_params - head_params) * T + 2.0 * head_params * 1 + attn_flops
    prefill = {"value": round(T / (pre_ms / 1e3), 1), "tokens": T, "ms": round(pre_ms, 3),
               "frac": round(flops / (pre_ms / 1e3) / (peak_tflops * 1e12), 4),
               "tflops": round(flops / (pre_ms / 1e3) / 1e12, 1), "peak_tflops": peak_tflops}
    print(f"[bench] prefill: {prefill}", file=sys.stderr, flush=True)
    fam_out = None
    if families:
        with OpLog(ops, runner.plan, events=True) as log:
            total = one("families")
        fam = {}
        for c in log.calls:
            f = fam.setdefault(family_of(c), {"ms": 0.0, "flops": 0.0, "bytes": 0, "calls": 0})
            f["ms"] += c["events"][0].elapsed_time(c["events"][1])
            f["calls"] += 1
            if c["op"] in PRODUCTS and c["weight_shape"]:
                f["flops"] += 2.0 * c["rows"] * c["weight_shape"][0] * c["weight_shape"][1]
            elif c["op"] in ("paged_attention", "decode_attention_fused"):
                f["flops"] += attn_flops / max(1, len(n_attn_sites))
            else:
                f["bytes"] += c["moved_bytes"]
        fam_out = {"ms_with_events": round(total, 3)}
        for name, f in sorted(fam.items(), key=lambda kv: -kv[1]["ms"]):
            row = {"ms": round(f["ms"], 3), "calls": f["calls"]}
            if f["flops"]:
                tf = f["flops"] / (f["ms"] / 1e3) / 1e12
                row.update(tflops=round(tf, 1), frac_peak=round(tf / peak_tflops, 3))
            else:
                gb = f["bytes"] / (f["ms"] / 1e3) / 1e9
                row.update(GBps=round(gb, 0), frac_hbm=round(gb / pk["hbm_gbs"], 3))
            fam_out[name] = row
    return prefill, fam_out


def reference_arm():
    """The reference is a Rust workspace (Cargo, candle); it has no Python package to
    install and no Rust toolchain exists here, so its arm cannot run."""
    print(json.dumps({"impl": "reference",
                      "unavailable": "Heyo-Computer/vapi is a Rust/Cargo workspace with no Python packaging; "
                                     "pip cannot install it offline and there is no cargo/rustc in the image"}),
          flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=32)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (0 = all)")
    ap.add_argument("--impl", default="vapi_b200", choices=["vapi_b200", "reference"])
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill", "serve", "trace"],
                    help="run just the headline decode point, just the prefill, (serve) continuous "
                         "batching of --requests requests with random prompt lengths through the engine loop, or "
                         "(trace) a few decode steps of a measuring build whose kernels stamp the device clock, "
                         "and print what one step's kernels did inside the captured graph")
    ap.add_argument("--sizes", default="1.2b", choices=["1.2b", "700m", "2.6b"], help="layer sizes of LFM2-<sizes>")
    ap.add_argument("--page-size", type=int, default=0, help="tokens per cache page (0: the engine's default)")
    ap.add_argument("--dtype", default="bfloat16", help="bfloat16 (serving) or float32 (the true 32-bit path)")
    ap.add_argument("--no-fp32", action="store_true", help="leave the float32 points out of the default run")
    ap.add_argument("--no-kernels", action="store_true", help="leave the decode step's kernel table (a second process) out")
    ap.add_argument("--rows-json", action="store_true", help="with --only trace: one JSON line of named kernels")
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--max-tokens", type=int, default=128)
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus %d is not supported" % args.gpus, flush=True)
        return 2
    if args.warmup < 3:
        args.warmup = 3
    return run(args)


if __name__ == "__main__":
    sys.exit(main())
