"""bin/trace_run against the plain implementation: every request whole, with its last 32
tokens decoded one by one, in portions of changing size down to two tokens, and mixed with
other requests in a pool so small that pages and state slots are used again; in float32 and
in bfloat16, for tiny configurations that differ in every size and option."""
import pytest
import torch

import plain_lfm2
import replay_util as ru
from conftest import TINY_A, TINY_A0, TINY_B, TINY_B0, TINY_C, TINY_D, TINY_E

pytestmark = pytest.mark.gpu

CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E, "A0": TINY_A0, "B0": TINY_B0}


def _requests(cfg, seed, lengths):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}


@pytest.fixture(scope="module")
def bf16_dirs(tmp_path_factory):
    """The tiny models with weights stored in bfloat16 (what a served checkpoint looks like)."""
    from vapi_b200.weights import write_random_model
    out = {}
    for name, seed in (("A", 10), ("B", 12), ("C", 14), ("D", 16), ("E", 18), ("A0", 20), ("B0", 22)):
        d = tmp_path_factory.mktemp(f"tiny{name}bf16")
        write_random_model(str(d), CONFIGS[name], seed, std=0.1 if name in "DE" else 0.2, norm_init="perturbed",
                           dtype=torch.bfloat16)
        out[name] = str(d)
    return out


def _full_trace(cfg, seed):
    """All the ways of cutting, one after the other, in a single run."""
    lengths = [1, 7, 33, 150, 97, 200, 64, 129, 70, 45]
    if cfg["max_position_embeddings"] < 200:                   # (the configuration with 128 positions)
        lengths = [1, 7, 33, 110, 97, 128, 64, 127, 70, 45]
    reqs = _requests(cfg, seed, lengths)
    tr = ru.Trace()
    ref_tokens = {}

    def use(tag, rid):
        ref_tokens[tag] = reqs[rid]
        return tag, reqs[rid]

    for rid in ("r0", "r1", "r2", "r3"):                       # alone and whole
        ru.whole(tr, *use(f"whole-{rid}", rid))
    for rid in ("r3", "r4", "r6", "r0"):                       # last 32 one by one
        ru.tail_decode(tr, *use(f"tail-{rid}", rid))
    ru.portions(tr, *use("cut-r5", "r5"), sizes=[2, 3, 64, 2, 17, 31, 2, 5, 62, 2])
    ru.portions(tr, *use("cut-r7", "r7"), sizes=[63, 2, 64, 1])     # boundaries on and beside a page edge
    ru.portions(tr, *use("cut2-r3", "r3"), sizes=[2])
    mix = {f"mix-{k}": v for k, v in reqs.items()}
    ref_tokens.update(mix)
    ru.mixed(tr, mix, seed=seed + 1)
    return tr, ref_tokens


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "A0", "B0"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_way_of_cutting(name, dtype, tiny_dirs, bf16_dirs, tmp_path):
    model_dir = tiny_dirs[name] if dtype == "float32" else bf16_dirs[name]
    plain = plain_lfm2.PlainLfm2(model_dir)
    tr, ref_tokens = _full_trace(CONFIGS[name], seed=100 + sum(map(ord, name)))
    ref = {k: plain.logits(v) for k, v in ref_tokens.items()}
    # the pool is exactly what the trace needs at its fullest, so pages are used again and again
    got = ru.run_trace(model_dir, dtype, tr, str(tmp_path / "out"))
    ok, msg = ru.compare(tr, got, ref, dtype)
    assert ok, msg
    total = sum(ru.round_up(len(v)) for v in ref_tokens.values())
    assert total > 3 * tr.peak_tokens, "the trace must need far more pages over time than the pool has"


def test_float32_checkpoint_served_in_bfloat16(tiny_dirs, tmp_path):
    """Weights stored in 32 bits stay 32-bit when serving in bfloat16: the run still works
    and stays within the bfloat16 limit."""
    plain = plain_lfm2.PlainLfm2(tiny_dirs["B"])
    reqs = _requests(TINY_B, 5, [90, 40])
    tr = ru.Trace()
    ru.tail_decode(tr, "r0", reqs["r0"], tail=8)
    ru.portions(tr, "r1", reqs["r1"], sizes=[2, 9])
    got = ru.run_trace(tiny_dirs["B"], "bfloat16", tr, str(tmp_path / "out"))
    ok, msg = ru.compare(tr, got, {k: plain.logits(v) for k, v in reqs.items()}, "bfloat16")
    assert ok, msg


def test_long_decoding_float32(tiny_dirs, tmp_path):
    """A short prompt and 300 tokens one by one: across several page edges, far from the start."""
    plain = plain_lfm2.PlainLfm2(tiny_dirs["A"])
    toks = _requests(TINY_A, 9, [330])["r0"]
    tr = ru.Trace()
    ru.tail_decode(tr, "r0", toks, tail=300)
    got = ru.run_trace(tiny_dirs["A"], "float32", tr, str(tmp_path / "out"))
    ok, msg = ru.compare(tr, got, {"r0": plain.logits(toks)}, "float32")
    assert ok, msg


def test_out_of_pages_is_an_error_not_a_wrong_result(tiny_dirs, tmp_path):
    toks = _requests(TINY_A, 3, [130])["r0"]
    tr = ru.Trace()
    ru.whole(tr, "r0", toks)
    with pytest.raises(RuntimeError, match="out of pages"):
        ru.run_trace(tiny_dirs["A"], "float32", tr, str(tmp_path / "out"), max_tokens=128)


@pytest.mark.parametrize("sizes", ["1.2b", "700m"])
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_layers_of_serving_size(sizes, dtype, tmp_path):
    """Three layers with the sizes of the 1.2B model (hidden 2048, 32 heads over 8 kv heads of 64,
    feed-forward 8192) and of the 700M model (hidden 1536, 24 heads, feed-forward 6912: three query
    heads per kv head, widths that are no power of two), conv - attention - conv: the shapes the
    serving kernels are tuned for, whole, in portions, token by token and mixed, against the plain
    model; with bfloat16 weights on the serving kernels, and with float32 weights on the true
    32-bit path, where the float32 limit holds at these widths too."""
    from conftest import serving_width_config
    from vapi_b200.weights import write_random_model
    cfg = serving_width_config(sizes)
    d = write_random_model(str(tmp_path / "m"), cfg, 3, std=0.02, norm_init="perturbed",
                           dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    plain = plain_lfm2.PlainLfm2(d)
    reqs = _requests(cfg, 8, [300, 40, 150, 20, 9, 25, 33, 12, 70, 3, 16, 48])
    tr = ru.Trace()
    ru.whole(tr, "whole-r0", reqs["r0"])
    ru.tail_decode(tr, "tail-r2", reqs["r2"], tail=6)
    ru.portions(tr, "cut-r0", reqs["r0"], sizes=[100, 2, 64, 17])
    mix = {f"mix-{k}": v for k, v in reqs.items()}
    ru.mixed(tr, mix, seed=4, max_live=12, decode_tail=8)      # up to 12 live: decode steps of 9..16 rows too
    ref_tokens = {"whole-r0": reqs["r0"], "tail-r2": reqs["r2"], "cut-r0": reqs["r0"], **mix}
    ref = {k: plain.logits(v) for k, v in ref_tokens.items()}
    got = ru.run_trace(d, dtype, tr, str(tmp_path / "out"), extra_args=["--max-requests", "16"])
    ok, msg = ru.compare(tr, got, ref, dtype, bf16_frac=0.02)
    assert ok, msg
