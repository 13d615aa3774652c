"""The engine loop, the sampler's host path and the Python entry point on a CPU, with the
plain restatements standing in for the kernels; and the plain implementation itself."""
import math

import numpy as np
import pytest
import torch

import plain_lfm2
from conftest import TINY_A, TINY_A0, TINY_B, TINY_B0
from vapi_b200.engine.engine import Engine
from vapi_b200.engine.runner import ModelRunner
from vapi_b200.engine.scheduler import SchedulerConfig
from vapi_b200.sampling.params import FinishReason, SamplingParams
from vapi_b200.sampling.sampler import SamplerState, host_sample


def _engine(model_dir, num_pages=16, page=16, max_requests=4, **sched):
    r = ModelRunner.from_dir(model_dir, dtype="float32", device="cpu", page_size=page, num_pages=num_pages,
                             max_requests=max_requests, max_batched_tokens=64)
    return Engine(r, SchedulerConfig(**sched), use_graphs=False)


def _prompts(cfg, seed, lens):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(8, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]


# ---- the plain implementation ----------------------------------------------------------
def test_plain_is_causal_and_stable_in_float64(tiny_dirs):
    p32 = plain_lfm2.PlainLfm2(tiny_dirs["B"])
    p64 = plain_lfm2.PlainLfm2(tiny_dirs["B"], dtype=torch.float64)
    toks = _prompts(TINY_B, 1, [40])[0]
    a, b = p32.logits(toks), p64.logits(toks)
    assert (a - b).abs().max() < 2e-4
    # a later token cannot change an earlier position
    toks2 = toks[:20] + [t ^ 1 for t in toks[20:]]
    # (within rounding: the CPU library may split a product differently from one call to the next)
    c = p32.logits(toks2)
    assert (c[:20] - a[:20]).abs().max() < 1e-5 and not torch.allclose(c[20:], a[20:], atol=1e-2)


def test_plain_shortconv_by_hand():
    c = dict(hidden=2, L=3, conv_bias=True)
    w = {"in_proj.weight": torch.eye(2).repeat(3, 1), "in_proj.bias": torch.tensor([0., 0., 1., 1., 0., 0.]),
         "conv.weight": torch.tensor([[[1., 10., 100.]], [[2., 20., 200.]]]), "conv.bias": torch.tensor([0.5, 0.5]),
         "out_proj.weight": torch.eye(2), "out_proj.bias": torch.zeros(2)}
    a = torch.tensor([[1., 1.], [2., 3.], [4., 5.]])
    # B = x = a, C = a + 1; g = a*a: [1,1],[4,9],[16,25]
    # conv[2] ch0 = 1*1 + 10*4 + 100*16 + .5 = 1641.5 ; ch1 = 2*1 + 20*9 + 200*25 + .5 = 5182.5
    # conv[0] ch0 = 100*1 + .5 ; conv[1] ch0 = 10*1 + 100*4 + .5
    y = plain_lfm2.shortconv(a, w, "", c)
    want = torch.tensor([[2 * 100.5, 2 * 200.5], [3 * 410.5, 4 * 1820.5], [5 * 1641.5, 6 * 5182.5]])
    assert torch.allclose(y, want)


def test_plain_rope_and_norm_by_hand():
    x = torch.tensor([[[1., 2., 3., 4.]]])                       # one token, one head, d = 4
    cos, sin = plain_lfm2.rope_tables(torch.tensor([0]), 4, 10000.0, torch.float32)
    assert torch.equal(plain_lfm2.rope(x, cos, sin), x)          # position 0 rotates nothing
    cos, sin = plain_lfm2.rope_tables(torch.tensor([1]), 4, 10000.0, torch.float32)
    y = plain_lfm2.rope(x, cos, sin)[0, 0]
    a0, a1 = 1.0, 1.0 / 100.0                                    # inv_freq = theta^(-0/4), theta^(-2/4)
    want = [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
            3 * math.cos(a0) + 1 * math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1)]
    assert torch.allclose(y, torch.tensor(want), atol=1e-6)
    n = plain_lfm2.rmsnorm(torch.tensor([3., 4.]), torch.tensor([2., 0.5]), 0.0)
    assert torch.allclose(n, torch.tensor([3 / math.sqrt(12.5) * 2, 4 / math.sqrt(12.5) * 0.5]))


# ---- the engine --------------------------------------------------------------------------
def test_greedy_generation_matches_the_plain_model(tiny_dirs, plain_kernels):
    plain = plain_lfm2.PlainLfm2(tiny_dirs["A"])
    eng = _engine(tiny_dirs["A"], prefill_chunk_tokens=7, max_context=128)
    prompts = _prompts(TINY_A, 1, [1, 7, 33])
    for i, p in enumerate(prompts):
        eng.admit(i, p, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    done = {f.request_id: f for f in eng.run()}
    for i, p in enumerate(prompts):
        assert done[i].tokens == plain.greedy(p, 8), f"request {i}"
        assert done[i].reason == FinishReason.LENGTH
    eng.runner.cache.check_invariants()
    assert eng.runner.cache.slots.num_free == 4


def test_the_two_described_tiny_workloads(tiny_dirs, plain_kernels):
    """The tiny configurations as the benchmark description words them, with its workloads: A with
    prompts of 1, 7 and 33 tokens (seed 1) and 16 greedy steps; B (one kv head of 16, vocabulary 512,
    256 positions, an untied head) with three requests of 5, 40 and 97 tokens as a mixed batch,
    prompts cut into portions of 16, sampled at temperature 0.8 with seed 3."""
    plain = plain_lfm2.PlainLfm2(tiny_dirs["A0"])
    eng = _engine(tiny_dirs["A0"], prefill_chunk_tokens=16, max_context=128)
    prompts = _prompts(TINY_A0, 1, [1, 7, 33])
    for i, p in enumerate(prompts):
        eng.admit(i, p, SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True))
    done = {f.request_id: f for f in eng.run()}
    assert [done[i].tokens for i in range(3)] == [plain.greedy(p, 16) for p in prompts]
    plain = plain_lfm2.PlainLfm2(tiny_dirs["B0"])
    eng = _engine(tiny_dirs["B0"], num_pages=24, prefill_chunk_tokens=16, max_context=256)
    prompts = _prompts(TINY_B0, 3, [5, 40, 97])
    for i, p in enumerate(prompts):
        eng.admit(i, p, SamplingParams(temperature=0.8, seed=3, max_tokens=6, ignore_eos=True))
    done = {f.request_id: f for f in eng.run()}
    assert [done[i].tokens for i in range(3)] == [plain.sample(p, 6, 0.8, 3) for p in prompts]
    assert eng.stats.steps > 7, "prompts were cut into portions and decoded beside one another"


def test_preemption_recomputes_to_the_same_tokens(tiny_dirs, plain_kernels):
    """A pool too small for both requests at once: one is preempted and recomputed, and
    both still produce what they produce alone."""
    plain = plain_lfm2.PlainLfm2(tiny_dirs["A"])
    prompts = _prompts(TINY_A, 2, [30, 28])
    eng = _engine(tiny_dirs["A"], num_pages=5, page=16, prefill_chunk_tokens=16, max_context=128)
    for i, p in enumerate(prompts):
        eng.admit(i, p, SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True))
    done = {f.request_id: f for f in eng.run()}
    assert eng.stats.preemptions > 0
    for i, p in enumerate(prompts):
        assert done[i].tokens == plain.greedy(p, 24)
    eng.runner.cache.check_invariants()


def test_a_failed_step_fails_requests_in_flight_and_the_engine_goes_on(tiny_dirs, plain_kernels):
    """Host-side fault injection (the reference's MockBackend::failing_at,
    crates/vapi-engine/src/backend.rs:446-450): the step function raises once."""
    plain = plain_lfm2.PlainLfm2(tiny_dirs["A"])
    eng = _engine(tiny_dirs["A"], max_context=128)
    real, calls = eng.step_fn, {"n": 0}

    def flaky(plan):
        calls["n"] += 1
        if calls["n"] == 2:
            raise RuntimeError("injected")
        return real(plan)

    eng.step_fn = flaky
    p = _prompts(TINY_A, 3, [5, 6])
    eng.admit("a", p[0], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    eng.admit("b", p[1], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    done = {f.request_id: f for f in eng.run()}
    assert done["a"].reason == FinishReason.ERROR and done["b"].reason == FinishReason.ERROR
    assert eng.stats.failed_steps == 1
    eng.runner.cache.check_invariants()
    assert eng.runner.cache.slots.num_free == 4 and eng.runner.cache.paged[0].pool.num_free == 16
    eng.admit("c", p[0], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    (c,) = eng.run()
    assert c.tokens == plain.greedy(p[0], 4)


def test_a_status_left_by_a_kernel_fails_the_step(tiny_dirs, plain_kernels):
    """A kernel that refuses an index or gives up a bounded wait records a status word and leaves
    its output unwritten.  The engine reads the word with the step's tokens: the step then counts
    as failed (requests in flight end with ``error``, everything goes back), the word is cleared,
    and the engine serves the next request.  The word is injected on the host here."""
    from vapi_b200.engine.runner import KernelRefusal, STATUS_NAMES
    plain = plain_lfm2.PlainLfm2(tiny_dirs["A"])
    eng = _engine(tiny_dirs["A"], max_context=128)
    p = _prompts(TINY_A, 3, [5, 6])
    eng.admit("a", p[0], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    eng.admit("b", p[1], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    eng.step()
    eng.runner.status[0] = 16
    done = {f.request_id: f for f in eng.run()}
    assert done["a"].reason == FinishReason.ERROR and done["b"].reason == FinishReason.ERROR
    assert eng.stats.failed_steps == 1 and "wait" in eng.last_error and 16 in STATUS_NAMES
    assert int(eng.runner.status[0]) == 0
    eng.runner.cache.check_invariants()
    assert eng.runner.cache.slots.num_free == 4 and eng.runner.cache.paged[0].pool.num_free == 16
    eng.admit("c", p[0], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    (c,) = eng.run()
    assert c.tokens == plain.greedy(p[0], 4) and c.reason == FinishReason.LENGTH
    eng.runner.status[0] = 4
    with pytest.raises(KernelRefusal, match="page id"):
        eng.runner.check_status()
    assert int(eng.runner.status[0]) == 0


def test_the_status_word_travels_with_the_sampled_tokens():
    """The sampler's pending result carries the word that stood in front of the tokens."""
    from vapi_b200.sampling.sampler import PendingSample, Sampler
    host = torch.tensor([16, 7, 8, 9], dtype=torch.int32)

    class Done:
        def synchronize(self):
            pass

    pending = PendingSample(3, host, Done(), with_status=True)
    assert Sampler("cpu").finish(pending) == [7, 8, 9] and pending.status == 16
    pending = PendingSample(3, host[1:], Done())
    assert Sampler("cpu").finish(pending) == [7, 8, 9] and pending.status == 0


def test_decode_buckets_stay_within_the_packers_capacity(tiny_dirs):
    """A request limit that is no power of two: the largest bucket is the limit itself, so the
    padded step of 40 live requests still fits the packer (48 sequences) instead of asking for 64."""
    r = ModelRunner.from_dir(tiny_dirs["A"], dtype="float32", device="cpu", page_size=16, num_pages=64,
                             max_requests=48, max_batched_tokens=64)
    assert r.graph_max_batch == 48
    assert [r._bucket(s) for s in (1, 3, 4, 17, 33, 40, 48)] == [1, 4, 4, 32, 48, 48, 48]
    r.packer.set_pad_pages(r.cache.set_aside_pages())
    for s in (3, 40):
        B = r._bucket(s)
        ctx = r.packer.pack([], r.dtype, n_cap=B, s_cap=B, width=r.packer.max_width)
        assert ctx.n == B and ctx.num_seqs == B


def test_failures_in_a_row_are_passed_on(tiny_dirs, plain_kernels):
    eng = _engine(tiny_dirs["A"], max_context=128)
    eng.max_step_failures = 2

    def broken(plan):
        raise RuntimeError("always")

    eng.step_fn = broken
    eng.admit("a", [9, 9], SamplingParams(max_tokens=2))
    eng.step()
    eng.admit("b", [9, 9], SamplingParams(max_tokens=2))
    with pytest.raises(RuntimeError, match="always"):
        eng.step()


def test_seeded_temperature_sampling_is_reproducible_and_independent_of_the_batch(tiny_dirs, plain_kernels):
    prompts = _prompts(TINY_B, 4, [5, 40, 97])
    sp = SamplingParams(temperature=0.8, max_tokens=6, seed=3, ignore_eos=True)

    def run(which):
        eng = _engine(tiny_dirs["B"], num_pages=24, prefill_chunk_tokens=16, max_context=256)
        for i in which:
            eng.admit(i, prompts[i], sp)
        return {f.request_id: f.tokens for f in eng.run()}

    together, alone = run([0, 1, 2]), run([1])
    assert together == run([0, 1, 2])
    assert together[1] == alone[1]


def test_python_entry_point(tiny_dirs, plain_kernels):
    from vapi_b200 import LLM
    plain = plain_lfm2.PlainLfm2(tiny_dirs["A"])
    llm = LLM(tiny_dirs["A"], dtype="f32", device="cpu", num_blocks=16, page_size=16, max_concurrent_seqs=4,
              max_batched_tokens=64, max_context=128, cuda_graphs=False)
    prompts = _prompts(TINY_A, 5, [3, 12])
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    assert [c.tokens for c in out] == [plain.greedy(p, 5) for p in prompts]
    assert out[0].finish_reason == "length" and out[0].prompt_tokens == 3


def test_python_entry_point_raises_when_a_step_failed(tiny_dirs, plain_kernels):
    from vapi_b200 import LLM
    llm = LLM(tiny_dirs["A"], dtype="f32", device="cpu", num_blocks=16, page_size=16, max_concurrent_seqs=4,
              max_batched_tokens=64, max_context=128, cuda_graphs=False)
    real, calls = llm.engine.step_fn, {"n": 0}

    def flaky(plan):
        calls["n"] += 1
        if calls["n"] == 2:
            raise RuntimeError("injected")
        return real(plan)

    llm.engine.step_fn = flaky
    prompts = _prompts(TINY_A, 5, [3, 12])
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    with pytest.raises(RuntimeError, match="2 of 2 requests ended in a failed step: RuntimeError: injected"):
        llm.generate(prompts, sp)
    # the engine goes on; a caller that wants the failed completions themselves can have them
    plain = plain_lfm2.PlainLfm2(tiny_dirs["A"])
    assert [c.tokens for c in llm.generate(prompts, sp)] == [plain.greedy(p, 5) for p in prompts]
    calls["n"] = 0
    out = llm.generate(prompts, sp, raise_on_error=False)
    assert [c.finish_reason for c in out] == ["error", "error"]


# ---- the sampler's host path -------------------------------------------------------------
def test_host_sampler_truncations():
    logits = np.array([0.0, 3.0, 2.9, -50.0, 1.0], dtype=np.float32)
    st = SamplerState(1)
    assert host_sample(logits, SamplingParams(temperature=0.0), st) == 1
    assert all(host_sample(logits, SamplingParams(temperature=1.0, top_k=1), st) == 1 for _ in range(20))
    seen = {host_sample(logits, SamplingParams(temperature=1.0, top_k=2), st) for _ in range(200)}
    assert seen == {1, 2}
    seen = {host_sample(logits, SamplingParams(temperature=1.0, min_p=0.5), st) for _ in range(200)}
    assert seen == {1, 2}
    seen = {host_sample(logits, SamplingParams(temperature=1.0, top_p=0.5), st) for _ in range(200)}
    assert seen == {1, 2}          # p(1) ~ 0.47 < 0.5, so the second token is needed to reach top_p
    a = [host_sample(logits, SamplingParams(temperature=1.5), SamplerState(7)) for _ in range(5)]
    b = [host_sample(logits, SamplingParams(temperature=1.5), SamplerState(7)) for _ in range(5)]
    assert a == b
    n, N = 0, 4000
    st = SamplerState(9)
    for _ in range(N):
        n += host_sample(logits, SamplingParams(temperature=1.0), st) == 1
    p1 = float(np.exp(3.0) / np.exp(logits.astype(np.float64)).sum())
    assert abs(n / N - p1) < 4 * math.sqrt(p1 * (1 - p1) / N)


def test_sampling_params_validation():
    for bad in (dict(temperature=2.5), dict(top_p=0.0), dict(min_p=1.5), dict(top_k=0), dict(max_tokens=0),
                dict(repetition_penalty=0.0)):
        with pytest.raises(ValueError):
            SamplingParams(**bad).validate()
    assert SamplingParams(temperature=0.0).is_greedy and not SamplingParams().is_greedy
    assert SamplingParams(temperature=0.7).device_drawable and not SamplingParams(temperature=0.7, top_k=5).device_drawable


def test_logprobs_are_the_models_own_distribution(tiny_dirs, plain_kernels):
    """``logprobs=k``: for every generated token its log-probability under the raw logits and the
    k most likely tokens, most likely first (crates/vapi-engine/src/sampler.rs:114-153), whatever
    temperature and penalties do to the choice."""
    plain = plain_lfm2.PlainLfm2(tiny_dirs["B"])
    eng = _engine(tiny_dirs["B"], max_context=128)
    p = _prompts(TINY_B, 7, [9])[0]
    eng.admit("g", p, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True, logprobs=3))
    eng.admit("t", p, SamplingParams(temperature=1.3, seed=4, presence_penalty=1.0, max_tokens=5, ignore_eos=True, logprobs=2))
    eng.admit("n", p, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    done = {f.request_id: f for f in eng.run()}
    assert done["n"].logprobs is None and done["n"].tokens == done["g"].tokens
    for rid, k in (("g", 3), ("t", 2)):
        f = done[rid]
        assert len(f.logprobs) == len(f.tokens) == 5
        text = list(p)
        for tok, lp in zip(f.tokens, f.logprobs):
            want = torch.log_softmax(plain.logits(text)[-1].double(), -1)
            assert lp.token == tok and abs(lp.logprob - float(want[tok])) < 1e-4
            top = torch.topk(want, k)
            assert [t for t, _ in lp.top] == top.indices.tolist()
            assert max(abs(a - float(b)) for (_, a), b in zip(lp.top, top.values)) < 1e-4
            text.append(tok)
    assert done["g"].logprobs[0].top[0][0] == done["g"].tokens[0]          # greedy takes the most likely token
    with pytest.raises(ValueError, match="logprobs"):
        SamplingParams(logprobs=21).validate()
    with pytest.raises(ValueError, match="n must"):
        SamplingParams(n=9).validate()


def test_row_logprobs_breaks_ties_by_the_lower_id():
    from vapi_b200.sampling.sampler import row_logprobs
    import numpy as np
    row = np.array([0.5, 2.0, 2.0, -1.0, 2.0, 0.5], dtype=np.float32)
    lse, top = row_logprobs(row, 4)
    assert [t for t, _ in top] == [1, 2, 4, 0]
    assert abs(lse - float(torch.logsumexp(torch.tensor(row), 0))) < 1e-6
    assert row_logprobs(row, 0)[1] == []


# ---- the bench's reading of the kernels' time stamps -----------------------------------------

def test_trace_table_takes_the_last_whole_step():
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location("bench", os.path.join(os.path.dirname(__file__), "..", "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)

    def ev(ns, kind, lib, blocks=4, threads=128):
        return {"ns": ns, "kind": kind, "library": lib, "blocks": blocks, "threads": threads}

    events = []
    for step in range(3):
        t = step * 1000
        events += [ev(t + 10, "start", "elementwise"), ev(t + 20, "released", "elementwise"),
                   ev(t + 15, "start", "gemv", 296, 256), ev(t + 120, "released", "gemv", 296, 256),
                   ev(t + 100, "start", "sampling", 8), ev(t + 400, "released", "sampling", 8)]
    events.sort(key=lambda e: e["ns"])
    rows = bench.trace_table(events)
    assert [r["library"] for r in rows] == ["elementwise", "gemv", "sampling"]
    assert rows[0]["at_us"] == 0 and rows[0]["until_next_us"] == pytest.approx(0.1)
    assert rows[1]["waited_us"] == pytest.approx(0.105) and rows[1]["until_next_us"] == pytest.approx(0.28)
    assert rows[2]["until_next_us"] is None
    assert bench.trace_table(events[:4]) == []
