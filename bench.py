#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at LFM2-1.2B sizes with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 4096] [--layers N]

One JSON line on stdout.  ``value`` is decoded tokens per second at the given batch, device-
timed over exactly K decode steps with CUDA events (each step: the packed index data goes
host->device, the captured decode graph replays, greedy tokens are chosen on the device).
``e2e`` is the same metric through the engine loop a user drives (scheduler, step, sampler,
host tokens in and out, wall clock).  ``prefill`` times one 2,048-token prompt in one step;
``roofline`` relates the decode step to the bytes it must read.  Peaks come from
MEASURED_PEAKS.json when the file is there, else from the fallback figures.

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


def model_numbers(runner):
    """Bytes of every weight a decode step reads once, and matrix-product flops per token."""
    import torch
    seen, wbytes, mm_params = set(), 0, 0
    plan = runner.plan

    def add(t, is_matrix):
        nonlocal wbytes, mm_params
        if t is None or t.data_ptr() in seen:
            return
        seen.add(t.data_ptr())
        wbytes += t.numel() * t.element_size()
        if is_matrix:
            mm_params += t.numel()

    for call in plan.order:
        blk = plan.layers[call.layer]
        for part in (blk.mixer, blk.ffn, blk.mixer_norm, blk.ffn_norm):
            for v in vars(part).values():
                if isinstance(v, torch.Tensor):
                    add(v, v.dim() == 2 and v.shape[0] > 8)
    add(plan.final_norm.weight, False)
    add(plan.head.weight, True)        # tied: the embedding table, read once by the head
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


def run(args):
    if args.only == "trace":          # a measuring build of every kernel library, named before the first import
        os.environ["VAPI_NVCC_FLAGS"] = (os.environ.get("VAPI_NVCC_FLAGS", "") + " -DVAPI_TRACE").strip()
    import torch
    from vapi_b200 import ops
    from vapi_b200.engine.engine import Engine
    from vapi_b200.engine.runner import ModelRunner
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
    pages = max_b * (-(-ctx_len // page)) + 8
    runner = ModelRunner.from_random(cfg, seed=0, dtype="bfloat16", device="cuda:0", num_pages=pages, page_size=page,
                                     max_requests=max_b, max_batched_tokens=8192, max_context=ctx_len + 256,
                                     watermark=0.0, validate=False)
    wbytes, mm_params = model_numbers(runner)
    gen = torch.Generator().manual_seed(1)
    vocab = cfg["vocab_size"]

    def fill(batch, length):
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

    def decode_steps(rcs, count, timed):
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

    def decode_point(batch, steps, warmup, clocks=None):
        start_len = ctx_len - (steps + warmup) - 1
        rcs = fill(batch, start_len)
        decode_steps(rcs, warmup, False)
        if clocks:
            clocks.start()
        before = ops.launch_count
        ms = decode_steps(rcs, steps, True)
        launches = ops.launch_count - before
        clk = clocks.stop() if clocks else None
        kv_bytes = sum(rc.num_tokens for rc in rcs) * runner.cache.bytes_per_token() + \
            batch * runner.cache.state_bytes_per_request()
        for rc in rcs:
            runner.cache.close(rc)
        return ms, launches, clk, kv_bytes

    if args.only == "prefill":
        return prefill_only(args, runner, mm_params, pk, gen, vocab, dev)
    if args.only == "trace":
        # the decode step as it runs inside its captured graph, from the kernels' own time stamps
        ops.trace_start()
        steps = min(args.steps, 8)
        ms, _, _, _ = decode_point(B, steps, min(args.warmup, 4))
        rows = trace_table(ops.trace_read())
        print(f"decode step, batch {B}, context {ctx_len}: {ms / steps:.4f} ms/step with the stamps on; one step's kernels in "
              f"the order in which their dependency waits returned", flush=True)
        print("   at us   library      blocks threads  waited us  until the next kernel's wait returns, us", flush=True)
        for r in rows:
            nxt = f"{r['until_next_us']:8.2f}" if r["until_next_us"] is not None else "       -"
            print(f"{r['at_us']:8.2f}   {r['library']:12s} {r['blocks']:6d} {r['threads']:7d}  {r['waited_us']:9.2f}  {nxt}", flush=True)
        return 0
    # ---- headline: decode at the given batch -----------------------------------------
    clocks = ClockSampler()
    ms, launches, clk, kv_bytes = decode_point(B, args.steps, args.warmup, clocks)
    ms_step = ms / args.steps
    value = B * args.steps / (ms / 1e3)
    print(f"[bench] decode b{B}: {value:.0f} tok/s, {ms_step:.3f} ms/step", file=sys.stderr, flush=True)
    step_bytes = wbytes + kv_bytes
    achieved = step_bytes / (ms_step / 1e3) / 1e9

    if args.only == "decode":
        print(json.dumps({"only": "decode", "value": round(value, 1), "ms_per_step": round(ms_step, 4),
                          "gpu_launches": launches, "roofline_frac": round(achieved / pk["hbm_gbs"], 4)}), flush=True)
        return 0
    # ---- other batch sizes ----------------------------------------------------------
    points = {}
    for b in (1, 64):
        st = max(16, min(128, args.steps // 2))
        m, _, _, _ = decode_point(b, st, max(3, min(16, args.warmup // 2)))
        points[f"decode_b{b}"] = round(b * st / (m / 1e3), 1)
        print(f"[bench] decode b{b}: {points[f'decode_b{b}']} tok/s", file=sys.stderr, flush=True)

    prefill = measure_prefill(runner, mm_params, pk, gen, vocab, dev)
    c = runner.plan.config
    n_attn = sum(1 for t in c.layer_types if t == "full_attention")

    # ---- end to end through the engine loop ----------------------------------------
    eng = Engine(runner, SchedulerConfig(max_concurrent_seqs=max_b, max_batched_tokens=8192,
                                         prefill_chunk_tokens=4096, max_context=ctx_len + 256), use_graphs=True)
    # requests finish their prompts at different steps, so leave room for the early ones
    start_len = ctx_len - (args.steps + args.warmup) - 2
    for i in range(B):
        prompt = torch.randint(0, vocab, (start_len,), generator=gen).tolist()
        eng.admit(("e2e", i), prompt, SamplingParams(temperature=0.0, max_tokens=args.steps + args.warmup + 128,
                                                     ignore_eos=True))
    while any(s.needs_prefill() for s in eng.scheduler.seqs.values()) or eng.scheduler.num_waiting:
        eng.step()
    for _ in range(args.warmup):
        eng.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    h2d = d2h = got = 0
    for _ in range(args.steps):
        out = eng.step()        # (the engine runs one step ahead: these are the tokens of the step before)
        got += len(out.new_tokens)
        h2d += runner.packer.h2d_bytes_last + eng.sampler.h2d_bytes_last
        d2h += eng.sampler.d2h_bytes_last
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    assert got == B * args.steps, (got, eng.stats, eng.last_error)
    e2e = {"value": round(got / e2e_s, 1), "unit": "tokens/s",
           "h2d_bytes_per_step": h2d // args.steps, "d2h_bytes_per_step": d2h // args.steps,
           "ms_per_step": round(e2e_s * 1e3 / args.steps, 4)}
    runner.check_status()
    st = eng.stats
    print(f"[bench] e2e: {e2e}; host ms/step over {st.steps} steps: schedule {st.schedule_ms / st.steps:.3f}, "
          f"forward(pack+launch) {st.forward_ms / st.steps:.3f}, sample(+wait for the GPU) {st.sample_ms / st.steps:.3f}, "
          f"commit {st.commit_ms / st.steps:.3f}", file=sys.stderr, flush=True)

    line = {
        "metric": "LFM2-%s decode tokens/s (batch %d, context %d), random weights" % (args.sizes.upper(), B, ctx_len),
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (seeded uniform-random token ids, random-init weights N(0, 0.02))",
        "impl": "vapi_b200",
        "config": {
            "model": "LFM2-%s sizes" % args.sizes.upper(), "global_batch": B, "seq_len": ctx_len, "parallelism": "single GPU",
            "layers": layers, "layers_of_configuration": full_layers, "attention_layers": n_attn,
            "hidden_size": c.hidden_size, "intermediate_size": c.intermediate_size, "vocab_size": c.vocab_size,
            "heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads, "head_dim": c.head_dim,
            "conv_L_cache": c.conv_L_cache, "page_size": page, "cuda_graphs": True,
            "l2": "inputs larger than L2 (weights %.2f GB per step)" % (wbytes / 1e9),
            "peaks": pk["source"],
        },
        "e2e": e2e,
        "gpu_launches": launches,
        "clocks": clk,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes)},
        "points": points,
    }
    print(json.dumps(line), flush=True)
    return 0


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


def measure_prefill(runner, mm_params, pk, gen, vocab, dev, warm=3, iters=5):
    """One 2,048-token prompt in one step, L2 flushed before each timed run."""
    import torch
    from vapi_b200.engine.step import StepEntry
    T = 2048
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    times = []
    for it in range(warm + iters):
        rc = runner.cache.open(("prefill", it))
        toks = torch.randint(0, vocab, (T,), generator=gen).tolist()
        assert runner.cache.reserve(rc, T)
        flush.zero_()                                   # larger than L2: nothing of the last run stays cached
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        runner.step([StepEntry(rc, toks, [T - 1])])
        e1.record()
        torch.cuda.synchronize()
        if it >= warm:
            times.append(e0.elapsed_time(e1))
        runner.cache.close(rc)
    pre_ms = sorted(times)[len(times) // 2]
    c = runner.plan.config
    n_attn = sum(1 for t in c.layer_types if t == "full_attention")
    head_params = runner.plan.head.weight.numel()
    flops = 2.0 * (mm_params - head_params) * T + 2.0 * head_params * 1 + \
        n_attn * 4.0 * c.num_attention_heads * c.head_dim * (T * (T + 1) / 2)
    prefill = {"value": round(T / (pre_ms / 1e3), 1), "tokens": T, "ms": round(pre_ms, 3),
               "frac": round(flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
               "tflops": round(flops / (pre_ms / 1e3) / 1e12, 1), "peak_tflops": pk["bf16_tflops"]}
    print(f"[bench] prefill: {prefill}", file=sys.stderr, flush=True)
    return prefill


def prefill_only(args, runner, mm_params, pk, gen, vocab, dev):
    p = measure_prefill(runner, mm_params, pk, gen, vocab, dev, warm=max(1, min(args.warmup, 3)), iters=max(1, min(args.steps, 5)))
    print(json.dumps({"only": "prefill", "prefill": p}), flush=True)
    return 0


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
