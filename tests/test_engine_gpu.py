"""On the GPU: greedy generation through the Python entry point against the plain model,
captured decode steps against eager ones, temperature sampling, each part alone against the
plain model's function for it, and a toy mixer with state of its own that is registered,
built and stepped without touching the package's files."""
import pytest
import torch

import plain_lfm2
from conftest import TINY_A, TINY_A0, TINY_B, TINY_B0, TINY_C, TINY_D

pytestmark = pytest.mark.gpu


def _prompts(cfg, seed, lens):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(8, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]


def _agrees_up_to_a_near_tie(plain, prompt, got, want, gap=0.5):
    """bfloat16 may part from the float32 tokens only where the plain top-1/top-2 gap is small
    (the reference's rule for real models, crates/vapi-backend-candle/tests/real_model.rs:336-341)."""
    for i, (a, b) in enumerate(zip(got, want)):
        if a != b:
            top = torch.topk(plain.logits(list(prompt) + want[:i])[-1], 2).values
            return float(top[0] - top[1]) < gap
    return True


@pytest.mark.parametrize("name,cfg", [("A", TINY_A), ("B", TINY_B), ("C", TINY_C)])
def test_greedy_generation_float32(name, cfg, tiny_dirs):
    from vapi_b200 import LLM, SamplingParams
    plain = plain_lfm2.PlainLfm2(tiny_dirs[name])
    prompts = _prompts(cfg, 1, [1, 7, 33, 70])
    for graphs in (False, True):
        llm = LLM(tiny_dirs[name], dtype="f32", num_blocks=24, max_concurrent_seqs=4, max_batched_tokens=64,
                  max_context=256, prefill_chunk_tokens=16, cuda_graphs=graphs)
        out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True))
        llm.runner.check_status()
        for p, c in zip(prompts, out):
            want = plain.greedy(p, 16)
            assert c.tokens == want or _agrees_up_to_a_near_tie(plain, p, c.tokens, want, gap=1e-3), (graphs, c.tokens, want)
        llm.runner.cache.check_invariants()
        if graphs:
            assert llm.runner._graphs, "pure decode steps must have gone through a captured graph"


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_the_two_described_tiny_workloads(tiny_dirs, dtype):
    """The tiny configurations as the benchmark description words them, with its workloads, through
    the entry point: A (prompts of 1, 7, 33 tokens, 16 greedy steps) and B (three requests of 5, 40
    and 97 tokens as a mixed batch, portions of 16, temperature 0.8 with seed 3).  In float32 the
    tokens are the plain model's; in bfloat16 (float32 checkpoint, bfloat16 activations and cache)
    they may part only at a near-tie of the plain model."""
    from vapi_b200 import LLM, SamplingParams
    plain = plain_lfm2.PlainLfm2(tiny_dirs["A0"])
    prompts = _prompts(TINY_A0, 1, [1, 7, 33])
    llm = LLM(tiny_dirs["A0"], dtype=dtype, num_blocks=8, max_concurrent_seqs=4, max_batched_tokens=64, max_context=128,
              prefill_chunk_tokens=16)
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True))
    llm.runner.check_status()
    for p, c in zip(prompts, out):
        want = plain.greedy(p, 16)
        assert c.tokens == want or _agrees_up_to_a_near_tie(plain, p, c.tokens, want, gap=1e-3 if dtype == "f32" else 0.5)
    plain = plain_lfm2.PlainLfm2(tiny_dirs["B0"])
    prompts = _prompts(TINY_B0, 3, [5, 40, 97])
    llm = LLM(tiny_dirs["B0"], dtype=dtype, num_blocks=8, max_concurrent_seqs=4, max_batched_tokens=64, max_context=256,
              prefill_chunk_tokens=16)
    out = llm.generate(prompts, SamplingParams(temperature=0.8, seed=3, max_tokens=10, ignore_eos=True))
    llm.runner.check_status()
    if dtype == "f32":
        assert [c.tokens for c in out] == [plain.sample(p, 10, 0.8, 3) for p in prompts]
    else:
        assert all(len(c.tokens) == 10 for c in out)
        again = llm.generate(prompts, SamplingParams(temperature=0.8, seed=3, max_tokens=10, ignore_eos=True))
        assert [c.tokens for c in again] == [c.tokens for c in out]


def test_greedy_generation_bfloat16(tiny_dirs, tmp_path):
    from vapi_b200 import LLM, SamplingParams
    from vapi_b200.weights import write_random_model
    d = write_random_model(str(tmp_path / "m"), TINY_B, 12, std=0.2, norm_init="perturbed", dtype=torch.bfloat16)
    plain = plain_lfm2.PlainLfm2(d)
    prompts = _prompts(TINY_B, 2, [5, 40, 97])
    llm = LLM(d, dtype="bf16", num_blocks=24, max_concurrent_seqs=4, max_batched_tokens=64, max_context=256,
              prefill_chunk_tokens=16)
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    for p, c in zip(prompts, out):
        assert _agrees_up_to_a_near_tie(plain, p, c.tokens, plain.greedy(p, 12)), (c.tokens,)


def test_captured_decode_equals_eager_decode(tiny_dirs):
    from vapi_b200.engine.runner import ModelRunner
    from vapi_b200.engine.step import StepEntry
    prompts = _prompts(TINY_B, 3, [20, 3, 64])
    outs = {}
    for graphs in (False, True):
        r = ModelRunner.from_dir(tiny_dirs["B"], dtype="float32", num_pages=16, max_requests=4, max_batched_tokens=128,
                                 max_context=256)
        rcs = []
        for i, p in enumerate(prompts):
            rc = r.cache.open(i)
            assert r.cache.reserve(rc, len(p))
            r.step([StepEntry(rc, p, [])])
            rcs.append(rc)
        rows = []
        for s in range(6):
            entries = []
            for j, rc in enumerate(rcs):
                assert r.cache.reserve(rc, rc.num_tokens + 1)
                entries.append(StepEntry(rc, [(7 * s + j) % 500], [0]))
            lg = r.step_decode_graph(entries) if graphs else r.step(entries)
            assert lg is not None
            rows.append(lg.clone().cpu())
        outs[graphs] = torch.stack(rows)
        r.check_status()
    assert (outs[True] - outs[False]).abs().max() < 1e-4


def test_temperature_sampling_is_seeded_and_batch_independent(tiny_dirs):
    from vapi_b200 import LLM, SamplingParams
    prompts = _prompts(TINY_B, 4, [5, 40, 97])
    sp = SamplingParams(temperature=0.8, max_tokens=10, seed=3, ignore_eos=True)

    def run(which):
        llm = LLM(tiny_dirs["B"], dtype="f32", num_blocks=24, max_concurrent_seqs=4, max_batched_tokens=64,
                  max_context=256, prefill_chunk_tokens=16)
        return {i: c.tokens for i, c in zip(which, llm.generate([prompts[i] for i in which], sp))}

    together = run([0, 1, 2])
    assert together == run([0, 1, 2])
    assert together[1] == run([1])[1]
    greedy = LLM(tiny_dirs["B"], dtype="f32", num_blocks=24, max_concurrent_seqs=4, max_batched_tokens=64,
                 max_context=256).generate([prompts[1]], SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    assert together[1] != greedy[0].tokens, "temperature 0.8 on a flat tiny model should not reproduce greedy"
    # the cuts (top-k, min-p, top-p) are made on the device too; top-k 1 leaves the most likely token
    tk = LLM(tiny_dirs["B"], dtype="f32", num_blocks=24, max_concurrent_seqs=4, max_batched_tokens=64, max_context=256)
    one = tk.generate([prompts[1]], SamplingParams(temperature=1.0, top_k=1, max_tokens=10, seed=1, ignore_eos=True))
    assert one[0].tokens == greedy[0].tokens


@pytest.mark.parametrize("ahead", [True, False])
def test_a_status_word_on_the_device_fails_the_step_and_is_cleared(tiny_dirs, ahead):
    """The status word reaches the host in the copy that brings the sampled tokens; a non-zero word
    fails the step like a step function that raised.  The word is written from the host here (a
    kernel writes it when it refuses an index or gives up a bounded wait): nothing on the device
    is made to go wrong."""
    from vapi_b200 import LLM, SamplingParams
    plain = plain_lfm2.PlainLfm2(tiny_dirs["B"])
    prompts = _prompts(TINY_B, 6, [5, 23])
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    llm = LLM(tiny_dirs["B"], dtype="f32", num_blocks=24, max_concurrent_seqs=4, max_batched_tokens=64, max_context=256,
              run_ahead=ahead)
    llm.runner.status.fill_(16)
    out = llm.generate(prompts, sp, raise_on_error=False)
    assert [c.finish_reason for c in out] == ["error", "error"]
    assert "wait" in llm.engine.last_error and llm.engine.stats.failed_steps == 1
    assert int(llm.runner.status.item()) == 0
    llm.runner.cache.check_invariants()
    out = llm.generate(prompts, sp)
    for p, c in zip(prompts, out):
        want = plain.greedy(p, 6)
        assert c.tokens == want or _agrees_up_to_a_near_tie(plain, p, c.tokens, want, gap=1e-3)


def test_the_collector_stays_out_of_graph_capture(tiny_dirs):
    """Freeing another runner's graphs (garbage in reference cycles dies whenever the collector
    happens to run) is not permitted while a stream captures and would lose the capture: the
    collector runs before a capture and is off inside it."""
    import gc
    from vapi_b200 import LLM, SamplingParams
    llm = LLM(tiny_dirs["B"], dtype="bf16", num_blocks=24, max_concurrent_seqs=4, max_batched_tokens=64, max_context=256)
    real, seen = llm.runner.forward, []

    def spy(ctx):
        if torch.cuda.is_current_stream_capturing():
            seen.append(gc.isenabled())
        return real(ctx)

    llm.runner.forward = spy
    out = llm.generate(_prompts(TINY_B, 4, [5, 9]), SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    assert all(len(c.tokens) == 6 for c in out)
    assert seen and not any(seen), "the decode graph was captured, with the collector off"
    assert gc.isenabled()


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_running_one_step_ahead_changes_no_token(tiny_dirs, dtype):
    """The engine enqueues a step before it has read the tokens of the step before it.  With
    stops in the middle of the text, different lengths, seeded temperature, late admissions and a
    pool so small that requests are preempted, every request must end with the tokens and the
    reason it has without running ahead."""
    from vapi_b200 import LLM, SamplingParams
    prompts = _prompts(TINY_B, 9, [5, 40, 97, 3, 18, 64])

    def run(ahead, params, blocks):
        llm = LLM(tiny_dirs["B"], dtype=dtype, num_blocks=blocks, page_size=16, max_concurrent_seqs=4,
                  max_batched_tokens=64, max_context=256, prefill_chunk_tokens=16, run_ahead=ahead)
        out = llm.generate(prompts, params)
        llm.runner.check_status()
        llm.runner.cache.check_invariants()
        assert all(g.pool.num_free + 1 >= g.pool.num_pages for g in llm.runner.cache.paged)   # one page is set aside
        return [(c.tokens, c.finish_reason) for c in out], llm.engine.stats

    free = [SamplingParams(temperature=0.0, max_tokens=20 + 3 * i, ignore_eos=True) for i in range(6)]
    base, st0 = run(False, free, 40)
    assert st0.ahead_steps == 0
    # stop ids taken from the middle of what is generated, so that requests end on a stop while
    # the step after it is already enqueued
    stops = [SamplingParams(temperature=0.0, max_tokens=20 + 3 * i, ignore_eos=True,
                            stop_token_ids=(base[i][0][7 + i],)) for i in range(6)]
    want, _ = run(False, stops, 40)
    assert any(r == "stop" for _, r in want) and all(len(t) <= 20 + 3 * i for i, (t, _) in enumerate(want))
    got, st = run(True, stops, 40)
    assert got == want and st.ahead_steps > 10
    # a pool that forces preemptions (recompute must not need a token that is still in flight)
    want_small, st_s = run(False, free, 13)
    got_small, st_a = run(True, free, 13)
    assert st_s.preemptions > 0 and got_small == want_small
    # seeded temperature on the device: the draw counters advance the same way
    temp = [SamplingParams(temperature=0.9, seed=11 + i, max_tokens=16, ignore_eos=True) for i in range(6)]
    assert run(True, temp, 40)[0] == run(False, temp, 40)[0]
    # the same with the distribution cut by top-k / top-p / min-p for some of the requests
    cut = [SamplingParams(temperature=1.1, seed=21 + i, max_tokens=16, ignore_eos=True, top_k=(20 if i % 2 else None),
                          top_p=(0.9 if i % 3 else 1.0), min_p=(0.02 if i == 4 else 0.0)) for i in range(6)]
    a, st_cut = run(True, cut, 40)
    assert a == run(False, cut, 40)[0] and st_cut.ahead_steps > 10
    assert a != run(True, temp, 40)[0]


def test_one_step_ahead_and_graphs_with_the_serving_kernels(tmp_path):
    """Head size 64 and bfloat16 weights: the captured decode step runs the weight-streaming
    products, the conv epilogue and the tensor-core attention.  Tokens must not depend on whether
    the engine runs ahead or uses graphs, and must follow the plain model up to near-ties."""
    from vapi_b200 import LLM, SamplingParams
    from vapi_b200.weights import write_random_model
    d = write_random_model(str(tmp_path / "m"), TINY_D, 21, std=0.1, norm_init="perturbed", dtype=torch.bfloat16)
    plain = plain_lfm2.PlainLfm2(d)
    prompts = _prompts(TINY_D, 5, [3, 70, 130, 18, 64])
    params = [SamplingParams(temperature=0.0, max_tokens=12 + 2 * i, ignore_eos=True) for i in range(5)]
    outs = {}
    for ahead, graphs in ((True, True), (False, True), (True, False), (False, False)):
        llm = LLM(d, dtype="bf16", num_blocks=24, max_concurrent_seqs=4, max_batched_tokens=256, max_context=256,
                  prefill_chunk_tokens=128, run_ahead=ahead, cuda_graphs=graphs)
        outs[(ahead, graphs)] = [c.tokens for c in llm.generate(prompts, params)]
        llm.runner.check_status()
        llm.runner.cache.check_invariants()
        assert (llm.engine.stats.ahead_steps > 0) == ahead
    assert outs[(True, True)] == outs[(False, True)] and outs[(True, False)] == outs[(False, False)]
    for p, got in zip(prompts, outs[(True, True)]):
        assert _agrees_up_to_a_near_tie(plain, p, got, plain.greedy(p, len(got))), got


@pytest.mark.parametrize("sizes", ["1.2b", "700m"])
def test_captured_decode_at_serving_widths(sizes, tmp_path):
    """Three layers of the serving models' widths in bfloat16 through the engine with captured
    graphs, 12 and then 24 live requests: the buckets of 16 and 32 sequences (the sixteen-warp
    weight-streaming product, the tcgen05 product, decode attention cut for the whole context,
    padding rows).  Tokens follow the plain model up to near-ties, and the logits of a captured
    step are those of an eager step within bfloat16 rounding."""
    from conftest import serving_width_config
    from vapi_b200 import LLM, SamplingParams
    from vapi_b200.engine.runner import ModelRunner
    from vapi_b200.engine.step import StepEntry
    from vapi_b200.weights import write_random_model
    cfg = serving_width_config(sizes)
    d = write_random_model(str(tmp_path / "m"), cfg, 7, std=0.02, norm_init="perturbed", dtype=torch.bfloat16)
    plain = plain_lfm2.PlainLfm2(d)
    lens = [9, 33, 64, 17, 5, 40, 65, 12, 3, 28, 50, 21] * 2
    prompts = _prompts(cfg, 11, lens)
    span = float(plain.logits(prompts[1]).max() - plain.logits(prompts[1]).min())
    for live in (12, 24):
        llm = LLM(d, dtype="bf16", num_blocks=80, max_concurrent_seqs=32, max_batched_tokens=2048, max_context=256,
                  prefill_chunk_tokens=512, cuda_graphs=True)
        out = llm.generate(prompts[:live], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
        llm.runner.check_status()
        bucket = 16 if live == 12 else 32
        assert llm.runner._graphs.get(bucket) is not None, f"decode steps of {live} requests run as a graph of {bucket}"
        for p, c in zip(prompts, out):
            assert _agrees_up_to_a_near_tie(plain, p, c.tokens, plain.greedy(p, 4), gap=0.03 * span), c.tokens
    # one decode step of 12 requests: captured against eager against the plain model
    rows = {}
    for graphs in (True, False):
        r = ModelRunner.from_dir(d, dtype="bfloat16", num_pages=40, max_requests=16, max_batched_tokens=1024, max_context=256)
        rcs = []
        for i, p in enumerate(prompts[:12]):
            rc = r.cache.open(i)
            assert r.cache.reserve(rc, len(p) + 1)
            rcs.append(rc)
        r.step([StepEntry(rc, p, []) for rc, p in zip(rcs, prompts[:12])])
        entries = [StepEntry(rc, [100 + i], [0]) for i, rc in enumerate(rcs)]
        lg = r.step_decode_graph(entries) if graphs else r.step(entries)
        assert lg is not None
        rows[graphs] = lg.float().cpu().clone()
        r.check_status()
    want = torch.stack([plain.logits(p + [100 + i])[-1] for i, p in enumerate(prompts[:12])])
    assert float((rows[True] - rows[False]).abs().max()) < 0.01 * span
    assert float((rows[True] - want).abs().max()) < 0.02 * span


@pytest.mark.parametrize("route", ["stream", "swiglu"])
def test_prompt_sized_steps_on_the_persistent_product(tmp_path, monkeypatch, route):
    """Prompt portions of 33 rows and more on csrc/linear_prompt.cu: every product of the step with
    its fused prologue and epilogue (the stream form: deferred norms, residual adds, SwiGLU), or the
    library's products with only the gate|up product and its SwiGLU on the own kernel (what prompts
    run on unless told otherwise).  Whole, cut into portions, and beside decode tokens of others."""
    from conftest import serving_width_config
    from vapi_b200 import ops
    from vapi_b200.engine.runner import ModelRunner
    from vapi_b200.engine.step import StepEntry
    from vapi_b200.weights import write_random_model
    cfg = serving_width_config("700m")
    d = write_random_model(str(tmp_path / "m"), cfg, 9, std=0.02, norm_init="perturbed", dtype=torch.bfloat16)
    plain = plain_lfm2.PlainLfm2(d)
    monkeypatch.setattr(ops, "PROMPT_MIN_ROWS", 33 if route == "stream" else 0)
    monkeypatch.setattr(ops, "PROMPT_SWIGLU_MIN_ROWS", 33)
    a, b, c = _prompts(cfg, 12, [300, 77, 140])
    want_a, want_b, want_c = plain.logits(a), plain.logits(b), plain.logits(c)
    span = float(want_a.max() - want_a.min())
    r = ModelRunner.from_dir(d, dtype="bfloat16", num_pages=24, max_requests=4, max_batched_tokens=1024, max_context=512)
    before = ops.launch_count
    ra, rb, rc = r.cache.open("a"), r.cache.open("b"), r.cache.open("c")
    assert r.cache.reserve(ra, 300) and r.cache.reserve(rb, 77) and r.cache.reserve(rc, 140)
    # a whole, with logits everywhere; then b cut 40 + 36 + 1 with c's portions beside it
    got = r.step([StepEntry(ra, a, list(range(300)))])
    assert float((got.float().cpu() - want_a).abs().max()) < 0.03 * span
    assert r.step([StepEntry(rb, b[:40], []), StepEntry(rc, c[:100], [])]) is None
    got = r.step([StepEntry(rb, b[40:76], [35]), StepEntry(rc, c[100:], [39])])
    assert float((got[0].float().cpu() - want_b[75]).abs().max()) < 0.03 * span
    assert float((got[1].float().cpu() - want_c[139]).abs().max()) < 0.03 * span
    got = r.step([StepEntry(rb, b[76:], [0])])
    assert float((got[0].float().cpu() - want_b[76]).abs().max()) < 0.03 * span
    r.check_status()
    assert "linear_prompt" in ops.loaded_libraries and ops.launch_count > before
    for x in (ra, rb, rc):
        r.cache.close(x)
    r.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_step_runs_on_the_callers_stream(tiny_dirs, dtype):
    """The kernels of a step launch on the stream that is current when the step begins (looked up
    once per step): a step made under another stream than the default one gives the same logits,
    and work queued on that stream before the step is waited for."""
    from vapi_b200.engine.runner import ModelRunner
    from vapi_b200.engine.step import StepEntry
    (prompt,) = _prompts(TINY_D, 41, [37])
    outs = []
    for side in (False, True):
        r = ModelRunner.from_dir(tiny_dirs["D"], dtype=dtype, num_pages=8, max_requests=2, max_batched_tokens=64, max_context=128)
        rc = r.cache.open("a")
        assert r.cache.reserve(rc, len(prompt) + 1)
        if side:
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                torch.cuda._sleep(20_000_000)                       # the step must queue behind this, on s
                r.step([StepEntry(rc, prompt[:30], [])])
                lg = r.step([StepEntry(rc, prompt[30:], [6])])
                tail = r.step([StepEntry(rc, [9], [0])])
            torch.cuda.current_stream().wait_stream(s)
        else:
            r.step([StepEntry(rc, prompt[:30], [])])
            lg = r.step([StepEntry(rc, prompt[30:], [6])])
            tail = r.step([StepEntry(rc, [9], [0])])
        torch.cuda.synchronize()
        r.check_status()
        outs.append((lg.float().cpu(), tail.float().cpu()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


def test_the_cache_is_sized_from_free_memory(tiny_dirs):
    """Without a page count the runner takes a fraction of the free device memory, less the state
    slots (crates/vapi-backend-candle/src/backend.rs:385-400), and never more pages than every
    request at full context could use."""
    from vapi_b200 import LLM, SamplingParams
    from vapi_b200.engine.runner import ModelRunner
    plain = plain_lfm2.PlainLfm2(tiny_dirs["D"])
    free, _ = torch.cuda.mem_get_info()
    fraction = 24e6 / free                                     # a budget of about 24 MB
    r = ModelRunner.from_dir(tiny_dirs["D"], dtype="bfloat16", max_requests=64, max_batched_tokens=256, max_context=512,
                             num_pages=None, kv_cache_fraction=fraction)
    pages = r.cache.paged[0].pool.num_pages
    page_bytes = r.cache.bytes_per_token() * r.cache.page_size
    state_bytes = r.cache.state_bytes_per_request() * (64 + 1)
    assert 0 < pages < 64 * 8, "the budget, not the cap, decided"
    assert pages * page_bytes + state_bytes <= 24e6 * 1.01 and (pages + 1) * page_bytes + state_bytes > 24e6 * 0.95
    assert r.cache.paged[0].tensor.numel() * r.cache.paged[0].tensor.element_size() == pages * page_bytes
    # a generous fraction is capped by what the requests could ever use
    r2 = ModelRunner.from_dir(tiny_dirs["D"], dtype="bfloat16", max_requests=4, max_batched_tokens=256, max_context=512,
                              num_pages=None, kv_cache_fraction=0.5)
    assert r2.cache.paged[0].pool.num_pages == 4 * 8
    llm = LLM(tiny_dirs["D"], dtype="f32", max_concurrent_seqs=4, max_batched_tokens=256, max_context=256,
              kv_cache_fraction=fraction)
    p = _prompts(TINY_D, 3, [30, 9])
    out = llm.generate(p, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    for q, c in zip(p, out):
        want = plain.greedy(q, 6)
        assert c.tokens == want or _agrees_up_to_a_near_tie(plain, q, c.tokens, want, gap=1e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_windowed_group_and_a_layer_that_reads_another_layers_cache(tmp_path, dtype):
    """A plan from the package's own parts that LFM2 does not use: an attention layer with a
    window of 40 keys (a cache group of its own, whose pages are given back as the window passes
    them), and a run-order entry that reads the cache another entry owns (its own keys and values
    are computed and dropped).  Whole, in portions, token by token, beside another request, with
    so few pages that released pages are used again, against a plain restatement."""
    from vapi_b200.config import Architecture, register_architecture, unregister_architecture
    from vapi_b200.engine.runner import ModelRunner
    from vapi_b200.engine.step import StepEntry
    from vapi_b200.models.plan import LayerCall, ModelPlan
    from vapi_b200.parts import (GQAttention, OutputHead, PreNormBlock, RMSNorm, RotaryEncoding, SwiGLU, TokenEmbedding)
    from vapi_b200.weights import write_random_model
    H, nh, nkv, hd, F, V, W, eps, theta = 64, 4, 2, 16, 96, 120, 40, 1e-5, 10000.0
    sub = {"mixer_norm": "n1.", "mixer": "att.", "ffn_norm": "n2.", "ffn": "ffn."}

    def plan(cfg):
        emb = TokenEmbedding(V, H, "emb.weight")
        att = lambda window: GQAttention(H, nh, nkv, hd, qk_norm_eps=eps, pos="rope", window=window)
        layers = [PreNormBlock(RMSNorm(H, eps), att(w), RMSNorm(H, eps), SwiGLU(H, F, {"gate": "w1", "up": "w3", "down": "w2"}), sub)
                  for w in (0, W, 0)]
        # entry 2 reads the cache that entry 0 owns
        return ModelPlan("ToyWindowForCausalLM", V, H, 512, emb, layers, ["l0.", "l1.", "l2."],
                         [LayerCall(0), LayerCall(1), LayerCall(2, cache_of=0)], RMSNorm(H, eps), "final.",
                         OutputHead(V, H, True, emb), position_encodings=[RotaryEncoding(hd, theta, 512, "rope")])

    def plain_logits(w, toks):
        c = dict(heads=nh, kv_heads=nkv, head_dim=hd, eps=eps, theta=theta)
        x = w["emb.weight"][torch.tensor(toks)]
        kv0 = None
        for l, window in enumerate((0, W, 0)):
            pre = f"l{l}."
            a = plain_lfm2.rmsnorm(x, w[pre + "n1.weight"], eps)
            q, k, v = plain_lfm2.attention_heads(a, w, pre + "att.", c)
            if l == 0:
                kv0 = (k, v)
            if l == 2:
                k, v = kv0
            x = x + plain_lfm2.attend(q, k, v, window) @ w[pre + "att.out_proj.weight"].T
            x = x + plain_lfm2.feed_forward(plain_lfm2.rmsnorm(x, w[pre + "n2.weight"], eps), w, pre + "ffn.")
        return plain_lfm2.rmsnorm(x, w["final.weight"], eps) @ w["emb.weight"].T

    register_architecture(Architecture("ToyWindowForCausalLM", ("toy_window",), lambda v: v, plan), replace=True)
    try:
        d = write_random_model(str(tmp_path / "toy"), {"architectures": ["ToyWindowForCausalLM"]}, 3, std=0.2,
                               norm_init="perturbed", dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
        w = plain_lfm2.read_weights(d)
        # 10 pages of 16 a group: the request of 150 tokens needs 10 in the group that keeps everything,
        # and the windowed group serves it and its neighbour out of pages that keep coming back
        r = ModelRunner.from_dir(d, dtype=dtype, num_pages=12, page_size=16, max_requests=3, max_batched_tokens=256,
                                 max_context=256)
        assert [g.spec.window for g in r.cache.paged] == [0, W] and [len(g.sites) for g in r.cache.paged] == [1, 1]
        toks = torch.randint(0, V, (150,), generator=torch.Generator().manual_seed(5)).tolist()
        want = plain_logits(w, toks)
        span = float(want.max() - want.min())
        tol = 1e-4 * max(1.0, span / 10) if dtype == "float32" else 0.04 * span
        a = r.cache.open("whole")
        assert r.cache.reserve(a, len(toks))
        got = r.step([StepEntry(a, toks, list(range(len(toks))))]).cpu()
        assert float((got - want).abs().max()) < tol
        assert r.cache.paged[1].pool.num_free > r.cache.paged[0].pool.num_free, "the window released pages"
        r.cache.close(a)
        b, other = r.cache.open("cut"), r.cache.open("other")
        rows, pos = [], 0
        sizes = [2, 47, 1, 16, 33, 3] + [1] * 48
        for q in sizes:
            entries = [StepEntry(b, toks[pos:pos + q], list(range(q)))]
            assert r.cache.reserve(b, pos + q)
            if other.num_tokens < 30 and r.cache.reserve(other, other.num_tokens + 2):
                entries.insert(0, StepEntry(other, [3, 4], []))
            rows.append(r.step(entries).cpu())
            pos += q
        assert pos == len(toks)
        assert float((torch.cat(rows) - want).abs().max()) < tol
        r.check_status()
        r.cache.close(b)
        r.cache.close(other)
        r.cache.check_invariants()
        assert all(g.pool.num_free == g.pool.num_pages for g in r.cache.paged)
    finally:
        unregister_architecture("ToyWindowForCausalLM")


def test_several_completions_per_prompt_and_logprobs(tiny_dirs):
    from vapi_b200 import LLM, SamplingParams
    prompts = _prompts(TINY_B, 8, [12, 30])
    llm = LLM(tiny_dirs["B"], dtype="f32", num_blocks=24, max_concurrent_seqs=4, max_batched_tokens=64, max_context=256)
    sp = SamplingParams(temperature=0.9, seed=40, n=3, max_tokens=8, ignore_eos=True)
    out = llm.generate(prompts, sp)
    assert [(c.index, c.prompt_tokens) for c in out] == [(0, 12), (1, 12), (2, 12), (0, 30), (1, 30), (2, 30)]
    assert len({tuple(c.tokens) for c in out[:3]}) > 1, "three seeds should not all give the same text"
    for i in range(3):       # completion i is what seed + i gives on its own
        alone = llm.generate([prompts[1]], SamplingParams(temperature=0.9, seed=40 + i, max_tokens=8, ignore_eos=True))
        assert alone[0].tokens == out[3 + i].tokens
    plain = plain_lfm2.PlainLfm2(tiny_dirs["B"])
    lp = llm.generate([prompts[0]], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True, logprobs=2))[0]
    text = list(prompts[0])
    for tok, rec in zip(lp.tokens, lp.logprobs):
        want = torch.log_softmax(plain.logits(text)[-1], -1)
        assert rec.token == tok and abs(rec.logprob - float(want[tok])) < 1e-3 and rec.top[0][0] == tok
        text.append(tok)


def test_randomized_serving_gives_the_same_tokens_however_it_is_scheduled(tiny_dirs):
    """120 requests with random lengths, limits, stop ids and samplers (greedy, temperature, top-p,
    top-k, min-p) through the float32 engine: running ahead or not, and a pool that holds
    everything or one so small that requests queue and are preempted, must not change one token."""
    import random
    from vapi_b200 import LLM, SamplingParams
    rng = random.Random(2)
    g = torch.Generator().manual_seed(3)
    prompts, params = [], []
    for _ in range(120):
        n = rng.choice([1, 2, 3, 5, 17, 40, 63, 64, 65, 100, 129, 200])
        prompts.append(torch.randint(3, TINY_D["vocab_size"], (n,), generator=g).tolist())
        kw = dict(max_tokens=rng.randint(1, 30), seed=rng.randint(0, 10 ** 6), ignore_eos=rng.random() < 0.5,
                  stop_token_ids=tuple(rng.sample(range(3, 1003), rng.choice([0, 0, 5, 50]))))
        kind = rng.choice(["greedy", "temp", "topp", "topk", "minp"])
        kw.update({"greedy": dict(temperature=0.0), "temp": dict(temperature=rng.uniform(0.3, 1.5)),
                   "topp": dict(temperature=1.0, top_p=rng.uniform(0.1, 0.99)),
                   "topk": dict(temperature=1.2, top_k=rng.randint(1, 100)),
                   "minp": dict(temperature=1.0, min_p=rng.uniform(0.01, 0.3), top_p=0.95)}[kind])
        params.append(SamplingParams(**kw))
    res, stats = {}, {}
    for ahead, blocks in ((False, 200), (True, 200), (True, 14), (False, 14)):
        llm = LLM(tiny_dirs["D"], dtype="f32", num_blocks=blocks, max_concurrent_seqs=16, max_batched_tokens=512,
                  max_context=320, prefill_chunk_tokens=96, run_ahead=ahead)
        res[(ahead, blocks)] = [(c.tokens, c.finish_reason) for c in llm.generate(prompts, params)]
        llm.runner.check_status()
        llm.runner.cache.check_invariants()
        stats[(ahead, blocks)] = llm.engine.stats
    assert stats[(True, 200)].ahead_steps > 50 and stats[(True, 14)].ahead_steps > 0
    assert stats[(False, 14)].steps > 1.5 * stats[(False, 200)].steps, "the small pool must make requests wait"
    assert any(r == "stop" for _, r in res[(False, 200)]) and any(r == "length" for _, r in res[(False, 200)])
    for key, got in res.items():
        bad = [i for i, (a, b) in enumerate(zip(res[(False, 200)], got)) if a != b]
        assert not bad, (key, bad[:5])


def test_penalties_give_the_tokens_of_the_plain_model_with_the_rule_applied_on_the_host(tiny_dirs):
    """Repetition, frequency and presence penalties over the prompt's and the generated tokens
    (crates/vapi-engine/src/sampler.rs:249-283): greedy generation with them must give exactly
    the tokens of the plain model whose logits get the rule applied on the host."""
    import plain_ops
    from vapi_b200 import LLM, SamplingParams
    plain = plain_lfm2.PlainLfm2(tiny_dirs["B"])
    prompts = _prompts(TINY_B, 6, [12, 30])
    prompts[0] = prompts[0][:6] * 2                            # repeated tokens in the prompt count too
    llm = LLM(tiny_dirs["B"], dtype="f32", num_blocks=8, max_concurrent_seqs=2, max_batched_tokens=64, max_context=128)
    base = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True))
    changed = 0
    for rep, freq, pres in ((1.0, 1.0, 2.0), (1.7, 0.0, 0.0), (0.8, 0.3, 0.5)):
        sp = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True, repetition_penalty=rep,
                            frequency_penalty=freq, presence_penalty=pres)
        out = llm.generate(prompts, sp)
        for p, c, b0 in zip(prompts, out, base):
            text, counts, want = list(p), {}, []
            for t in p:
                counts[t] = counts.get(t, 0) + 1
            for _ in range(24):
                row = plain.logits(text)[-1:].clone()
                toks = sorted(counts)
                plain_ops.apply_penalties(row, torch.zeros(len(toks), dtype=torch.int32), torch.tensor(toks, dtype=torch.int32),
                                          torch.tensor([float(counts[t]) for t in toks]), torch.tensor([rep]),
                                          torch.tensor([freq]), torch.tensor([pres]))
                nxt = int(torch.argmax(row[0]))
                want.append(nxt)
                text.append(nxt)
                counts[nxt] = counts.get(nxt, 0) + 1
            assert c.tokens == want or _agrees_up_to_a_near_tie(plain, p, c.tokens, want, gap=1e-3), (rep, freq, pres)
            changed += c.tokens != b0.tokens
    assert changed >= 4, "the penalties must change what is generated"


# ---- each part alone -----------------------------------------------------------------------
def _ctx_for(n, S, cu, klens, positions, page_table=None, slots=None, state_slots=None, dtype=torch.float32):
    from vapi_b200.engine.step import GroupMeta, StepContext
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    tok_seq = []
    for s in range(S):
        tok_seq += [s] * (cu[s + 1] - cu[s])
    groups = [GroupMeta(i32(slots), i32(page_table))] if page_table is not None else []
    return StepContext(n=n, num_seqs=S, num_rows=0, max_q=max(cu[s + 1] - cu[s] for s in range(S)), max_k=max(klens),
                       tokens=i32([0] * n), positions=i32(positions), tok_seq=i32(tok_seq), cu_q=i32(cu),
                       seqlens_k=i32(klens), state_slots=i32(state_slots or [0] * S), logits_rows=None,
                       groups=groups, dtype=dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_parts_alone(dtype):
    """Norm, position encoding, attention, short conv, feed-forward and the block, each built
    from sizes alone (no model configuration), against the plain model's function."""
    from vapi_b200.parts import (CacheView, GQAttention, PreNormBlock, RMSNorm, RotaryEncoding, ShortConv, SwiGLU)
    torch.manual_seed(0)
    H, nh, nkv, d, F, L, T, eps, theta = 80, 5, 1, 32, 112, 4, 23, 1e-6, 5e4
    tol = dict(atol=2e-4, rtol=2e-4) if dtype == torch.float32 else dict(atol=6e-2, rtol=6e-2)
    c = dict(hidden=H, heads=nh, kv_heads=nkv, head_dim=d, eps=eps, theta=theta, L=L, conv_bias=True)
    w = {k: (torch.randn(s) * 0.2).to(dtype).float() for k, s in {
        "a.q_proj.weight": (nh * d, H), "a.k_proj.weight": (nkv * d, H), "a.v_proj.weight": (nkv * d, H),
        "a.out_proj.weight": (H, nh * d), "c.in_proj.weight": (3 * H, H), "c.out_proj.weight": (H, H),
        "f.w1.weight": (F, H), "f.w3.weight": (F, H), "f.w2.weight": (H, F)}.items()}
    w.update({"a.q_layernorm.weight": 1 + 0.1 * torch.randn(d), "a.k_layernorm.weight": 1 + 0.1 * torch.randn(d),
              "c.in_proj.bias": 0.2 * torch.randn(3 * H), "c.conv.weight": 0.5 * torch.randn(H, 1, L),
              "c.conv.bias": 0.2 * torch.randn(H), "c.out_proj.bias": 0.2 * torch.randn(H),
              "n1.weight": 1 + 0.1 * torch.randn(H), "n2.weight": 1 + 0.1 * torch.randn(H)})
    dev = {k: (v.cuda().to(dtype) if v.dim() == 2 and "conv" not in k else v.cuda()) for k, v in w.items()}
    x = torch.randn(T, H)
    a = x.to(dtype).float()

    page, pages = 16, 4
    ctx = _ctx_for(T, 1, [0, T], [T], list(range(T)), page_table=[[2, 0, 3, 1]],
                   slots=[[2, 0, 3, 1][p // page] * page + p % page for p in range(T)], dtype=dtype)
    rope = RotaryEncoding(d, theta, 4096)
    ctx.pos["rope"] = rope.prepare(ctx)
    cr, sr = plain_lfm2.rope_tables(torch.arange(T), d, theta, torch.float32)
    torch.testing.assert_close(ctx.pos["rope"][0].cpu(), cr, atol=1e-5, rtol=0)

    att = GQAttention(H, nh, nkv, d, qk_norm_eps=eps, pos="rope")
    att.bind(dev, "a.", dtype)
    kv = torch.zeros(pages, 2, nkv, page, d, dtype=dtype, device="cuda")
    got = att.forward(a.cuda().to(dtype), ctx, CacheView("paged", kv, ctx.groups[0], True))
    torch.testing.assert_close(got.float().cpu(), plain_lfm2.attention(a, w, "a.", c), **tol)

    conv = ShortConv(H, L, bias=True)
    conv.bind(dev, "c.", dtype)
    state = torch.full((2, L - 1, H), 5.0, dtype=dtype, device="cuda")
    got = conv.forward(a.cuda().to(dtype), ctx, CacheView("state", state, None, True))
    torch.testing.assert_close(got.float().cpu(), plain_lfm2.shortconv(a, w, "c.", c), **tol)

    ffn = SwiGLU(H, F)
    ffn.bind(dev, "f.", dtype)
    got = ffn.forward(a.cuda().to(dtype), ctx)
    torch.testing.assert_close(got.float().cpu(), plain_lfm2.feed_forward(a, w, "f."), **tol)

    norm = RMSNorm(H, eps)
    norm.bind(dev, "n1.", dtype)
    xs = x.clone().cuda()
    got = norm.apply(xs, None, dtype)
    torch.testing.assert_close(got.float().cpu(), plain_lfm2.rmsnorm(x, w["n1.weight"], eps), **tol)

    # the block: conv mixer + feed-forward around the float32 stream, pending delta handed on
    blk = PreNormBlock(RMSNorm(H, eps), ShortConv(H, L, bias=True), RMSNorm(H, eps), SwiGLU(H, F),
                       {"mixer_norm": "n1.", "mixer": "c.", "ffn_norm": "n2.", "ffn": "f."})
    blk.bind(dev, "", dtype)
    xs = x.clone().cuda()
    delta = blk.forward(xs, None, ctx, CacheView("state", torch.zeros_like(state), None, True))
    x1 = x + plain_lfm2.shortconv(plain_lfm2.rmsnorm(x, w["n1.weight"], eps), w, "c.", c)
    want = x1 + plain_lfm2.feed_forward(plain_lfm2.rmsnorm(x1, w["n2.weight"], eps), w, "f.")
    torch.testing.assert_close((xs + delta.float()).cpu(), want, **(tol if dtype == torch.float32 else dict(atol=0.15, rtol=6e-2)))


# ---- a toy mixer with state of its own --------------------------------------------------------
def _whole_cut_and_token_by_token(r, toks, vocab, limit, graphs):
    """One request whole in one step (more rows than the few-row route takes), then the same
    tokens in portions beside another request, the last ones one by one (through captured decode
    steps when ``graphs``); returns the worst difference between the two, which must stay below
    ``limit`` times the logit range."""
    from vapi_b200.engine.step import StepEntry
    n = len(toks)
    a = r.cache.open("whole")
    assert r.cache.reserve(a, n)
    whole = r.step([StepEntry(a, toks, list(range(n)))]).cpu()
    r.cache.close(a)
    b, other = r.cache.open("cut"), r.cache.open("other")       # `cut` lands in the slot `whole` used
    rows, pos = [], 0
    for q in (2, 1, 9, 1, 1, 16, 3):
        assert r.cache.reserve(b, pos + q) and r.cache.reserve(other, other.num_tokens + 2)
        out = r.step([StepEntry(other, [5, 6], []), StepEntry(b, toks[pos:pos + q], list(range(q)))])
        rows.append(out.cpu())
        pos += q
    used_graph = 0
    while pos < n:                                             # the rest token by token, two requests a step
        assert r.cache.reserve(b, pos + 1) and r.cache.reserve(other, other.num_tokens + 1)
        entries = [StepEntry(other, [7], [0]), StepEntry(b, toks[pos:pos + 1], [0])]
        out = r.step_decode_graph(entries) if graphs else None
        used_graph += out is not None
        if out is None:
            out = r.step(entries)
        rows.append(out[1:2].clone().cpu())
        pos += 1
    if graphs:
        assert used_graph > 0, "decode steps must have gone through a captured graph"
    r.check_status()
    span = float(whole.max() - whole.min())
    worst = float((torch.cat(rows) - whole).abs().max())
    assert worst < limit * max(span, 1.0), (worst, span)
    return whole


@pytest.mark.parametrize("dtype,hidden", [("float32", 48), ("bfloat16", 64)])
def test_a_toy_mixer_with_its_own_state_can_be_registered_built_and_stepped(tmp_path, dtype, hidden):
    """A running-mean mixer defined here: state = (sum of inputs so far) per request.  It gets
    a state slot from the cache manager, a registry entry, an architecture of its own, and
    runs through the package's step function, portions and decode tokens alike; the
    package's files are not touched.  Its math is plain torch on the device, which is the
    toy's own business; everything around it is the engine.

    In bfloat16 (widths that the package's own decode products take) steps of few rows run the
    blocks in their stream form: the toy mixer has none, so it is run the ordinary way between the
    package's feed-forwards, which add into the stream themselves; captured decode steps too."""
    from vapi_b200.config import Architecture, register_architecture, unregister_architecture
    from vapi_b200.engine.runner import ModelRunner
    from vapi_b200.models.plan import LayerCall, ModelPlan
    from vapi_b200.parts import (Mixer, OutputHead, PreNormBlock, RMSNorm, StateSpec, SwiGLU, TensorSpec,
                                 TokenEmbedding, register_mixer, make_part, MIXERS)
    from vapi_b200.weights import write_random_model

    class RunningMean(Mixer):
        def __init__(self, hidden):
            self.hidden = hidden

        def cache_spec(self):
            return StateSpec("running_sum", (self.hidden,), torch.float32)

        def tensor_specs(self, prefix):
            return [TensorSpec(prefix + "gain", (self.hidden,), role="vector", init="ones")]

        def bind(self, tensors, prefix, dtype):
            self.gain = tensors[prefix + "gain"]

        def forward(self, a, ctx, cache):
            if ctx.max_q == 1:               # one token a sequence: no host round trip, so a graph can hold it
                slots, first = ctx.state_slots.long(), (ctx.positions == 0)[:, None]
                run = torch.where(first, torch.zeros_like(a, dtype=torch.float32), cache.tensor[slots]) + a.float()
                cache.tensor.index_copy_(0, slots, run)
                return (run / (ctx.positions + 1)[:, None] * self.gain).to(a.dtype)
            out = torch.empty_like(a)
            cu, pos, slots = ctx.cu_q.tolist(), ctx.positions.tolist(), ctx.state_slots.tolist()
            for s in range(ctx.num_seqs):
                r0, r1 = cu[s], cu[s + 1]
                st = cache.tensor[slots[s]]
                base = st.clone() if pos[r0] > 0 else torch.zeros_like(st)     # position 0: nothing before
                run = base + torch.cumsum(a[r0:r1].float(), 0)
                cnt = torch.arange(pos[r0] + 1, pos[r0] + 1 + (r1 - r0), device=a.device).unsqueeze(1)
                out[r0:r1] = (run / cnt * self.gain).to(a.dtype)
                st.copy_(run[-1])
            return out

    register_mixer("toy_running_mean", RunningMean, replace=True)

    def plan(cfg):
        H, V = cfg["hidden_size"], cfg["vocab_size"]
        emb = TokenEmbedding(V, H, "emb.weight")
        layers = [PreNormBlock(RMSNorm(H, 1e-5), make_part(MIXERS, "toy_running_mean", hidden=H), RMSNorm(H, 1e-5),
                               SwiGLU(H, cfg["ff"]), {"mixer_norm": "n1.", "mixer": "mix.", "ffn_norm": "n2.", "ffn": "ffn."})
                  for _ in range(2)]
        # the run order names layer 0 twice: shared weights, a state of its own at each call site
        return ModelPlan("ToyForCausalLM", V, H, 512, emb, layers, ["l0.", "l1."],
                         [LayerCall(0), LayerCall(1), LayerCall(0)], RMSNorm(H, 1e-5), "final.",
                         OutputHead(V, H, True, emb))

    register_architecture(Architecture("ToyForCausalLM", ("toy",), lambda v: v, plan), replace=True)
    try:
        cfg = {"architectures": ["ToyForCausalLM"], "vocab_size": 100, "hidden_size": hidden, "ff": 64}
        d = write_random_model(str(tmp_path / "toy"), cfg, 0, std=0.3, norm_init="perturbed",
                               dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
        toks = torch.randint(0, 100, (45,), generator=torch.Generator().manual_seed(0)).tolist()
        r = ModelRunner.from_dir(d, dtype=dtype, num_pages=4, max_requests=3, max_batched_tokens=64, max_context=128)
        assert len(r.cache.state) == 1 and r.cache.state[0].tensor.shape == (4, 3, hidden) and not r.cache.paged
        if dtype == "float32":
            _whole_cut_and_token_by_token(r, toks, 100, 1e-5, graphs=False)
        else:
            from vapi_b200 import ops
            assert ops.few_rows_applies(2, r.plan.layers[0].ffn.w_gate_up), "the package's own product takes the feed-forward"
            got = _whole_cut_and_token_by_token(r, toks, 100, 0.03, graphs=True)
            # and the bfloat16 run stays near the same model in float32
            r32 = ModelRunner.from_dir(d, dtype="float32", num_pages=4, max_requests=3, max_batched_tokens=64, max_context=128)
            want = _whole_cut_and_token_by_token(r32, toks, 100, 1e-5, graphs=True)
            assert float((got - want).abs().max()) < 0.04 * float(want.max() - want.min())
    finally:
        unregister_architecture("ToyForCausalLM")
        MIXERS.pop("toy_running_mean", None)


# ---- a toy mixer that pages one row per token ---------------------------------------------------
def test_a_toy_mixer_that_pages_one_row_per_token_through_the_pools(tmp_path):
    """A causal convolution that keeps its input rows in the paged cache instead of a state slot
    (the reference's own layout for its conv layers, ``LayerLayout::Rows``,
    crates/vapi-backend-candle/src/cache.rs:22-45): one buffer of one row of the hidden width per
    token, with a window so that pages come back.  The cache manager lays the pages out from the
    description alone; the mixer reads earlier rows through the block table.  Defined here,
    registered, built and stepped (whole, portions, captured decode steps) without a change to
    the package."""
    from vapi_b200.config import Architecture, register_architecture, unregister_architecture
    from vapi_b200.engine.runner import ModelRunner
    from vapi_b200.models.plan import LayerCall, ModelPlan
    from vapi_b200.parts import (MIXERS, CacheView, Mixer, OutputHead, PagedSpec, PreNormBlock, RMSNorm, SwiGLU, TensorSpec,
                                 TokenEmbedding, make_part, register_mixer)
    from vapi_b200.weights import write_random_model
    L = 4

    class PagedRowsConv(Mixer):
        def __init__(self, hidden, taps):
            self.hidden, self.L = hidden, taps

        def cache_spec(self):
            return PagedSpec.rows(self.hidden, window=self.L)

        def tensor_specs(self, prefix):
            return [TensorSpec(prefix + "taps", (self.L, self.hidden), role="vector")]

        def bind(self, tensors, prefix, dtype):
            self.taps = tensors[prefix + "taps"]

        def forward(self, a, ctx, cache):
            rows = cache.buffers["row"]                              # [pages, 1, page_size, hidden]
            page = rows.shape[2]
            table = rows.view(-1, self.hidden)                       # row of (page, offset) at page * page_size + offset
            if cache.write:
                table.index_copy_(0, cache.group.slot_mapping.long(), a)
            pos, seq = ctx.positions.long(), ctx.tok_seq.long()
            out = self.taps[self.L - 1] * a.float()
            for k in range(1, self.L):                               # the row k positions back, through the block table
                q = (pos - k).clamp(min=0)
                slot = cache.group.block_table[seq, q // page].long() * page + q % page
                out = out + torch.where((pos - k >= 0)[:, None], self.taps[self.L - 1 - k] * table[slot].float(), 0.0)
            return out.to(a.dtype)

    register_mixer("toy_paged_rows_conv", PagedRowsConv, replace=True)

    def plan(cfg):
        H, V = cfg["hidden_size"], cfg["vocab_size"]
        emb = TokenEmbedding(V, H, "emb.weight")
        layers = [PreNormBlock(RMSNorm(H, 1e-5), make_part(MIXERS, "toy_paged_rows_conv", hidden=H, taps=L), RMSNorm(H, 1e-5),
                               SwiGLU(H, 64), {"mixer_norm": "n1.", "mixer": "mix.", "ffn_norm": "n2.", "ffn": "ffn."})
                  for _ in range(2)]
        return ModelPlan("ToyRowsForCausalLM", V, H, 512, emb, layers, ["l0.", "l1."], [LayerCall(0), LayerCall(1)],
                         RMSNorm(H, 1e-5), "final.", OutputHead(V, H, True, emb))

    register_architecture(Architecture("ToyRowsForCausalLM", ("toy_rows",), lambda v: v, plan), replace=True)
    try:
        cfg = {"architectures": ["ToyRowsForCausalLM"], "vocab_size": 100, "hidden_size": 48}
        d = write_random_model(str(tmp_path / "toy"), cfg, 0, std=0.3, norm_init="perturbed")
        # the mixer alone against the convolution written out
        r = ModelRunner.from_dir(d, dtype="float32", num_pages=6, page_size=16, max_requests=3, max_batched_tokens=64,
                                 max_context=128)
        assert len(r.cache.paged) == 1 and r.cache.paged[0].spec.window == L
        assert r.cache.paged[0].tensor.shape == (2, 6, 16 * 48), "two call sites, pages of 16 rows of 48"
        mixer = r.plan.layers[0].mixer
        T = 21
        a = torch.randn(T, 48, device="cuda")
        ctx = _ctx_for(T, 1, [0, T], [T], list(range(T)), page_table=[[3, 1]], slots=[[3, 1][p // 16] * 16 + p % 16 for p in range(T)])
        got = mixer.forward(a, ctx, CacheView("paged", r.cache.site_tensor(0), ctx.groups[0], True, r.cache.site_buffers(0),
                                              r.cache.site_spec(0)))
        want = torch.zeros_like(a)
        for t in range(T):
            for k in range(L):
                if t - k >= 0:
                    want[t] += mixer.taps[L - 1 - k] * a[t - k]
        assert float((got - want).abs().max()) < 1e-5
        # the model through the step function: 45 tokens need 3 pages at once only if nothing came back
        toks = torch.randint(0, 100, (45,), generator=torch.Generator().manual_seed(0)).tolist()
        _whole_cut_and_token_by_token(r, toks, 100, 1e-5, graphs=True)
        r.cache.check_invariants()
    finally:
        unregister_architecture("ToyRowsForCausalLM")
        MIXERS.pop("toy_paged_rows_conv", None)


# ---- a toy feed-forward with routing and a toy position encoding -----------------------------
@pytest.mark.parametrize("dtype,hidden", [("float32", 48), ("bfloat16", 64)])
def test_a_toy_routed_feed_forward_and_a_toy_position_encoding_can_be_registered_built_and_stepped(tmp_path, dtype, hidden):
    """Two more kinds of part defined here, neither of them a model of anyone's: a feed-forward
    that routes each token to one of several small experts (router logits and softmax in
    float32), and a position encoding that hands mixers a table of sines which a toy mixer adds to
    its input.  They sit in one plan beside the package's own attention (with its rotary
    encoding: two position encodings in one model), in layers of different kinds, and are stepped
    whole, in portions and token by token through the package's step function.

    In bfloat16 the attention layer runs in its stream form beside a feed-forward that has none,
    and the toy mixer beside the package's SwiGLU, in eager and in captured decode steps."""
    from vapi_b200.config import Architecture, register_architecture, unregister_architecture
    from vapi_b200.engine.runner import ModelRunner
    from vapi_b200.models.plan import LayerCall, ModelPlan
    from vapi_b200.parts import (FEED_FORWARDS, MIXERS, POSITION_ENCODINGS, FeedForward, GQAttention, Mixer, OutputHead,
                                 PositionEncoding, PreNormBlock, RMSNorm, RotaryEncoding, SwiGLU, TensorSpec,
                                 TokenEmbedding, make_part, register_feed_forward, register_mixer,
                                 register_position_encoding)
    from vapi_b200.weights import write_random_model

    class TopOneExperts(FeedForward):
        def __init__(self, hidden, width, experts):
            self.hidden, self.width, self.experts = hidden, width, experts

        def tensor_specs(self, prefix):
            return [TensorSpec(prefix + "router", (self.experts, self.hidden)),
                    TensorSpec(prefix + "up", (self.experts * self.width, self.hidden)),
                    TensorSpec(prefix + "down", (self.experts * self.hidden, self.width))]

        def bind(self, tensors, prefix, dtype):
            self.router = tensors[prefix + "router"].float()
            self.up = tensors[prefix + "up"].view(self.experts, self.width, self.hidden)
            self.down = tensors[prefix + "down"].view(self.experts, self.hidden, self.width)

        def forward(self, f, ctx):
            prob = torch.softmax(f.float() @ self.router.t(), dim=-1)              # routing in float32
            top_p, top_e = prob.max(dim=-1)
            out = torch.zeros_like(f)
            for e in range(self.experts):          # (every expert on every token, then masked: a toy may be wasteful)
                h = torch.relu(f @ self.up[e].t())
                y = ((h @ self.down[e].t()).float() * top_p[:, None]).to(f.dtype)
                out = torch.where((top_e == e)[:, None], y, out)
            return out

    class SineTable(PositionEncoding):
        def __init__(self, hidden, name="sines"):
            self.hidden, self.name = hidden, name

        def tensor_specs(self, prefix):
            return []

        def bind(self, tensors, prefix, dtype):
            pass

        def prepare(self, ctx):
            freq = torch.arange(1, self.hidden + 1, device=ctx.positions.device, dtype=torch.float32) / self.hidden
            return torch.sin(ctx.positions.float()[:, None] * freq[None, :])

    class AddPositions(Mixer):
        def __init__(self, hidden, pos):
            self.hidden, self.pos = hidden, pos

        def tensor_specs(self, prefix):
            return [TensorSpec(prefix + "gain", (self.hidden,), role="vector", init="ones")]

        def bind(self, tensors, prefix, dtype):
            self.gain = tensors[prefix + "gain"]

        def forward(self, a, ctx, cache):
            return ((a.float() + ctx.pos[self.pos]) * self.gain).to(a.dtype)

    register_feed_forward("toy_top_one_experts", TopOneExperts, replace=True)
    register_position_encoding("toy_sine_table", SineTable, replace=True)
    register_mixer("toy_add_positions", AddPositions, replace=True)

    def plan(cfg):
        H, V, E = cfg["hidden_size"], cfg["vocab_size"], cfg["experts"]
        emb = TokenEmbedding(V, H, "emb.weight")
        sub = {"mixer_norm": "n1.", "mixer": "mix.", "ffn_norm": "n2.", "ffn": "ffn."}
        layers = [
            PreNormBlock(RMSNorm(H, 1e-5), make_part(MIXERS, "toy_add_positions", hidden=H, pos="sines"), RMSNorm(H, 1e-5),
                         make_part(FEED_FORWARDS, "toy_top_one_experts", hidden=H, width=40, experts=E), sub),
            PreNormBlock(RMSNorm(H, 1e-6), GQAttention(H, 4, 1, 16, qk_norm_eps=1e-6, pos="rope"), RMSNorm(H, 1e-6),
                         make_part(FEED_FORWARDS, "toy_top_one_experts", hidden=H, width=40, experts=E), sub),
            PreNormBlock(RMSNorm(H, 1e-5), make_part(MIXERS, "toy_add_positions", hidden=H, pos="sines"), RMSNorm(H, 1e-5),
                         SwiGLU(H, 96), sub),
        ]
        return ModelPlan("ToyRoutedForCausalLM", V, H, 512, emb, layers, ["l0.", "l1.", "l2."],
                         [LayerCall(0), LayerCall(1), LayerCall(2)], RMSNorm(H, 1e-5), "final.",
                         OutputHead(V, H, True, emb),
                         position_encodings=[RotaryEncoding(16, 10000.0, 512, "rope"),
                                             make_part(POSITION_ENCODINGS, "toy_sine_table", hidden=H)])

    register_architecture(Architecture("ToyRoutedForCausalLM", ("toy_routed",), lambda v: v, plan), replace=True)
    try:
        cfg = {"architectures": ["ToyRoutedForCausalLM"], "vocab_size": 90, "hidden_size": hidden, "experts": 3}
        d = write_random_model(str(tmp_path / "toy"), cfg, 1, std=0.3, norm_init="perturbed",
                               dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
        kw = dict(num_pages=8, page_size=16, max_requests=3, max_batched_tokens=64, max_context=128)
        r = ModelRunner.from_dir(d, dtype=dtype, **kw)
        assert len(r.cache.paged) == 1 and not r.cache.state            # only the attention layer owns a cache
        toks = torch.randint(0, 90, (45,), generator=torch.Generator().manual_seed(2)).tolist()
        # the routed feed-forward really routes: more than one expert is in use on these tokens
        ffn = r.plan.layers[0].ffn
        x = r.plan.embedding.forward(type("C", (), {"tokens": torch.tensor(toks, dtype=torch.int32, device="cuda"),
                                                     "status": None})())
        used = torch.softmax(x.float() @ ffn.router.t(), -1).argmax(-1).unique().numel()
        assert used >= 2
        if dtype == "float32":
            _whole_cut_and_token_by_token(r, toks, 90, 2e-5, graphs=False)
        else:
            got = _whole_cut_and_token_by_token(r, toks, 90, 0.03, graphs=True)
            r32 = ModelRunner.from_dir(d, dtype="float32", **kw)
            want = _whole_cut_and_token_by_token(r32, toks, 90, 2e-5, graphs=True)
            # (a token whose two best experts are nearly tied may be routed differently in bfloat16:
            # compare the bulk, not the worst row)
            close = ((got - want).abs().amax(dim=1) < 0.04 * float(want.max() - want.min())).float().mean()
            assert float(close) > 0.9, float(close)
    finally:
        unregister_architecture("ToyRoutedForCausalLM")
        MIXERS.pop("toy_add_positions", None)
        FEED_FORWARDS.pop("toy_top_one_experts", None)
        POSITION_ENCODINGS.pop("toy_sine_table", None)
