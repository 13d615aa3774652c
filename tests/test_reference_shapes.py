"""The reference's own model tests, restated for this engine.

The reference checks LFM2 on a tiny fixture (crates/vapi-backend-candle/src/models/lfm2.rs:910-1025
and crates/vapi-backend-candle/tests/tiny_backends.rs:38-175): logits at all 18 positions of a fixed
prompt, one decode token against the cache, the prompt cut at every position 1..17 with the first
portion asking for nothing, one request's decode token beside another's whole prompt, bfloat16
within 5 % of the logit range, and greedy ids through the scheduler with prompts cut into portions
of 7, with and without captured graphs.

Its fixture has the shape below (tools/gen_lfm2_goldens.py:26-49: five layers conv, conv, attention,
conv, attention; theta 1e7 under ``rope_parameters``; weights N(0, 0.2) with norm weights 1 + 0.1 N)
and its golden logits lie in tests/goldens/lfm2-tiny.json, but the weights they were computed from
are drawn by a model class of the transformers package, which these tests may not import.  So the
same shapes, the same prompt and the same kind of weights are compared with the plain model of
``plain_lfm2`` instead of with the golden file.
"""
import pytest
import torch

import plain_lfm2
from vapi_b200.engine.runner import ModelRunner
from vapi_b200.engine.step import StepEntry

# tools/gen_lfm2_goldens.py:21-23, 27-35
PROMPT = [5, 17, 3, 42, 8, 9, 60, 33, 21, 7, 11, 2, 19, 44, 58, 13, 25, 31]
NEXT = 23
FIXTURE_SHAPE = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 256, "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 5,
    "num_attention_heads": 4, "num_key_value_heads": 2, "max_position_embeddings": 256,
    "layer_types": ["conv", "conv", "full_attention", "conv", "full_attention"],
    "conv_L_cache": 3, "conv_bias": False, "block_auto_adjust_ff_dim": False, "norm_eps": 1e-5,
    "tie_word_embeddings": True, "bos_token_id": 1, "eos_token_id": 2, "pad_token_id": 0,
    "rope_parameters": {"rope_type": "default", "rope_theta": 10000000.0},
}


@pytest.fixture(scope="module")
def fixture_dir(tmp_path_factory):
    from vapi_b200.weights import write_random_model
    d = tmp_path_factory.mktemp("lfm2-tiny-shape")
    return write_random_model(str(d), FIXTURE_SHAPE, 0, std=0.2, norm_init="perturbed", dtype=torch.float32)


def _runner(model_dir, dtype, device):
    return ModelRunner.from_dir(model_dir, dtype=dtype, device=device, page_size=16, num_pages=8, max_requests=4,
                                max_batched_tokens=64, max_context=256)


def _step(r, rc, tokens, want):
    assert r.cache.reserve(rc, rc.num_tokens + len(tokens))
    return r.step([StepEntry(rc, tokens, want)])


def _reference_shapes(model_dir, dtype, device, limit):
    plain = plain_lfm2.PlainLfm2(model_dir)
    n = len(PROMPT)
    full = plain.logits(PROMPT)
    decode = plain.logits(PROMPT + [NEXT])[-1]
    span = float(full.max() - full.min())
    tol = limit(span)

    def close(got, want, what):
        d = float((got.float().cpu() - want).abs().max())
        assert d < tol, f"{what}: max abs diff {d:.3e}, limit {tol:.3e}"

    # all positions, then the decode token against the cache (lfm2.rs:910-935)
    r = _runner(model_dir, dtype, device)
    rc = r.cache.open("a")
    close(_step(r, rc, PROMPT, range(n)), full, "full prompt")
    close(_step(r, rc, [NEXT], [0])[0], decode, "decode")
    r.cache.close(rc)
    # the prompt cut at every position; the first portion asks for nothing (lfm2.rs:937-953)
    for split in range(1, n):
        rc = r.cache.open(f"s{split}")
        assert _step(r, rc, PROMPT[:split], []) is None
        close(_step(r, rc, PROMPT[split:], range(n - split)), full[split:], f"prefill split at {split}")
        r.cache.close(rc)
    # A's decode token beside B's whole prompt (lfm2.rs:956-1002)
    b = PROMPT[::-1]
    want_b = plain.logits(b)[-1]
    ra, rb = r.cache.open("A"), r.cache.open("B")
    _step(r, ra, PROMPT, [])
    assert r.cache.reserve(ra, n + 1) and r.cache.reserve(rb, n)
    got = r.step([StepEntry(ra, [NEXT], [0]), StepEntry(rb, b, [n - 1])])
    close(got[0], decode, "A's decode in the mixed batch")
    close(got[1], want_b, "B's prefill in the mixed batch")
    r.cache.close(ra)
    r.cache.close(rb)
    r.cache.check_invariants()
    if device != "cpu":
        r.check_status()


def _greedy_through_the_scheduler(model_dir, dtype, device, graphs, near_tie_gap):
    """Greedy ids through the entry point with prompts cut into portions of 7
    (crates/vapi-backend-candle/tests/tiny_backends.rs:38-175)."""
    from vapi_b200 import LLM, SamplingParams
    plain = plain_lfm2.PlainLfm2(model_dir)
    llm = LLM(model_dir, dtype=dtype, device=device, num_blocks=8, page_size=16, max_concurrent_seqs=4,
              max_batched_tokens=64, max_context=256, prefill_chunk_tokens=7, cuda_graphs=graphs)
    prompts = [PROMPT, PROMPT[::-1], PROMPT[:5]]
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True))
    for p, c in zip(prompts, out):
        want = plain.greedy(p, 16)
        for i, (a, b) in enumerate(zip(c.tokens, want)):
            if a != b:
                top = torch.topk(plain.logits(list(p) + want[:i])[-1], 2).values
                assert float(top[0] - top[1]) < near_tie_gap, (c.tokens, want)
                break
    return [c.tokens for c in out]


def test_reference_shapes_on_the_host_logic(fixture_dir, plain_kernels):
    _reference_shapes(fixture_dir, "float32", "cpu", lambda span: 1e-4)
    _greedy_through_the_scheduler(fixture_dir, "f32", "cpu", False, 1e-3)


@pytest.mark.gpu
def test_reference_shapes_float32(fixture_dir):
    _reference_shapes(fixture_dir, "float32", "cuda", lambda span: 1e-4 * max(1.0, span / 10.0))


@pytest.mark.gpu
def test_reference_shapes_bfloat16(fixture_dir):
    # the reference's rule for this fixture in bfloat16: 5 % of the logit range (lfm2.rs:1004-1025)
    _reference_shapes(fixture_dir, "bfloat16", "cuda", lambda span: 0.05 * span)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_greedy_ids_through_the_scheduler_with_and_without_graphs(fixture_dir, dtype):
    gap = 1e-3 if dtype == "f32" else 0.5
    eager = _greedy_through_the_scheduler(fixture_dir, dtype, "cuda", False, gap)
    graphs = _greedy_through_the_scheduler(fixture_dir, dtype, "cuda", True, gap)
    if dtype == "f32":
        assert graphs == eager
