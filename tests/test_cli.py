"""``python -m vapi_b200`` as a user runs it (crates/vapi-core/src/cli.rs:26-56,
crates/vapi-worker/src/main.rs:24-52): the model folder by flag, by a TOML file named with ``-c``
and with ``$VAPI_CONFIG``, flags winning over the file, prompts from flags and from standard
input, random weights from a config.json, and the errors that end with exit code 2."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_lfm2
from conftest import ROOT, TINY_A, TINY_D


def _run(args, stdin=None, env=None, cwd=None):
    e = dict(os.environ)
    e["PYTHONPATH"] = ROOT + os.pathsep + e.get("PYTHONPATH", "")
    e.pop("VAPI_CONFIG", None)
    e.update(env or {})
    return subprocess.run([sys.executable, "-m", "vapi_b200"] + list(args), input=stdin, capture_output=True, text=True,
                          env=e, cwd=cwd, timeout=600)


def _prompts(cfg, seed, lens):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(8, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]


# ---- errors: nothing here needs a device ---------------------------------------------------
def test_an_unknown_argument_ends_with_code_2_and_is_named(tmp_path):
    p = _run(["--path", "x", "--no-such-flag", "1"], cwd=str(tmp_path))
    assert p.returncode == 2 and "--no-such-flag" in p.stderr
    p = _run(["--max-cont", "5"], cwd=str(tmp_path))          # abbreviations are not accepted either
    assert p.returncode == 2 and "--max-cont" in p.stderr


def test_configuration_errors_end_with_code_2(tmp_path):
    bad = tmp_path / "bad.toml"
    bad.write_text("[model]\npath = 'x'\nblocks = 3\n")
    p = _run(["-c", str(bad), "--prompt-ids", "1,2"], cwd=str(tmp_path))
    assert p.returncode == 2 and "unknown key `blocks`" in p.stderr
    p = _run(["-c", str(tmp_path / "absent.toml"), "--prompt-ids", "1,2"], cwd=str(tmp_path))
    assert p.returncode == 2 and "does not exist" in p.stderr
    p = _run(["--prompt-ids", "1,2"], cwd=str(tmp_path))
    assert p.returncode == 2 and "no model" in p.stderr
    p = _run(["--path", "x"], stdin="", cwd=str(tmp_path))
    assert p.returncode == 2 and "no prompts" in p.stderr
    p = _run(["--random-weights", "1", "--prompt-ids", "1,2"], cwd=str(tmp_path))
    assert p.returncode == 2 and "--config-json" in p.stderr
    p = _run(["--path", "x", "--kv-cache-fraction", "1.5", "--prompt-ids", "1"], cwd=str(tmp_path))
    assert p.returncode == 2 and "kv_cache_fraction" in p.stderr
    # ./vapi.toml is picked up when nothing else names a file
    (tmp_path / "vapi.toml").write_text("[queue]\nurl = 'x'\n")
    p = _run(["--prompt-ids", "1"], cwd=str(tmp_path))
    assert p.returncode == 2 and "unknown section [queue]" in p.stderr


# ---- generation -------------------------------------------------------------------------------
@pytest.mark.gpu
def test_model_by_flag_prompts_by_flag(tiny_dirs, tmp_path):
    plain = plain_lfm2.PlainLfm2(tiny_dirs["A"])
    prompts = _prompts(TINY_A, 21, [4, 19])
    args = ["--path", tiny_dirs["A"], "--dtype", "f32", "--num-blocks", "8", "--max-context", "128", "--max-concurrent-seqs", "4",
            "--max-batched-tokens", "64", "--prefill-chunk-tokens", "8", "--max-tokens", "7", "--stats"]
    for p in prompts:
        args += ["--prompt-ids", ",".join(map(str, p))]
    r = _run(args, cwd=str(tmp_path))
    assert r.returncode == 0, r.stderr[-2000:]
    recs = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert [x["tokens"] for x in recs] == [plain.greedy(p, 7) for p in prompts]
    assert [x["prompt_tokens"] for x in recs] == [4, 19] and all(x["finish_reason"] == "length" for x in recs)
    stats = json.loads(r.stderr.strip().splitlines()[-1])
    assert stats["tokens_out"] == 14 and stats["failed_steps"] == 0


@pytest.mark.gpu
def test_model_by_toml_prompts_by_stdin_and_flags_win_over_the_file(tiny_dirs, tmp_path):
    plain = plain_lfm2.PlainLfm2(tiny_dirs["A"])
    prompts = _prompts(TINY_A, 22, [3, 11, 30])
    toml = tmp_path / "serve.toml"
    toml.write_text(f"[model]\npath = '{tiny_dirs['A']}'\ndtype = 'f32'\nnum_blocks = 8\nmax_context = 4\ncuda_graphs = true\n"
                    "[worker]\nmax_concurrent_seqs = 4\nmax_batched_tokens = 64\nprefill_chunk_tokens = 16\n[cache]\nwatermark = 0.0\n")
    stdin = "".join(json.dumps(p) + "\n" for p in prompts)
    # the file's max_context of 4 would refuse every prompt; the flag wins
    r = _run(["-c", str(toml), "--max-context", "128", "--max-tokens", "5"], stdin=stdin, cwd=str(tmp_path))
    assert r.returncode == 0, r.stderr[-2000:]
    recs = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert [x["tokens"] for x in recs] == [plain.greedy(p, 5) for p in prompts]
    # the same file through the environment; a flag can switch the file's graphs off again
    r = _run(["--max-context", "128", "--max-tokens", "5", "--no-cuda-graphs", "--prompt-ids", ",".join(map(str, prompts[1]))],
             env={"VAPI_CONFIG": str(toml)}, cwd=str(tmp_path))
    assert r.returncode == 0, r.stderr[-2000:]
    (rec,) = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert rec["tokens"] == plain.greedy(prompts[1], 5)
    # without the flag the file's limit holds: the prompt is refused
    r = _run(["--max-tokens", "5", "--prompt-ids", ",".join(map(str, prompts[1]))], env={"VAPI_CONFIG": str(toml)}, cwd=str(tmp_path))
    assert r.returncode == 2 and "context limit" in r.stderr


@pytest.mark.gpu
def test_random_weights_from_a_config_json(tmp_path):
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(TINY_D))
    prompt = ",".join(map(str, _prompts(TINY_D, 23, [12])[0]))
    args = ["--random-weights", "5", "--config-json", str(cfg), "--dtype", "bf16", "--num-blocks", "8", "--max-context", "256",
            "--max-concurrent-seqs", "4", "--max-batched-tokens", "64", "--temperature", "0.7", "--seed", "9", "--max-tokens", "6",
            "--n", "2", "--prompt-ids", prompt, "--prompt-ids", prompt]
    r = _run(args, cwd=str(tmp_path))
    assert r.returncode == 0, r.stderr[-2000:]
    recs = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(recs) == 4 and [x["index"] for x in recs] == [0, 1, 0, 1]
    assert all(len(x["tokens"]) == 6 and all(0 <= t < TINY_D["vocab_size"] for t in x["tokens"]) for x in recs)
    # the same prompt, seed and completion index give the same tokens; another index another seed
    assert recs[0]["tokens"] == recs[2]["tokens"] and recs[1]["tokens"] == recs[3]["tokens"]
