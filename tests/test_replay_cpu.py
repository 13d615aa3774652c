"""The host side of trace replay on a CPU: bin/trace_run's own code, the cache manager, the
packer and the step function run as they are, with the plain restatements standing in for
the CUDA kernels.  What is checked is bookkeeping: positions, pages, slots, state carried
across portions, reuse of pages and slots."""
import importlib.machinery
import importlib.util
import io
import json
import os
import sys

import numpy as np
import pytest
import torch

import plain_lfm2
import replay_util as ru
from conftest import TINY_A, TINY_B


def _load_trace_run():
    loader = importlib.machinery.SourceFileLoader("trace_run_script", ru.TRACE_RUN)
    spec = importlib.util.spec_from_loader("trace_run_script", loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    return mod


def _run_in_process(monkeypatch, capsys, model_dir, tr, out_dir, max_tokens):
    mod = _load_trace_run()
    monkeypatch.setattr(sys, "stdin", io.StringIO("".join(json.dumps(s) + "\n" for s in tr.steps)))
    rc = mod.main(["--model", model_dir, "--dtype", "float32", "--out", out_dir, "--max-tokens", str(max_tokens),
                   "--device", "cpu"])
    done = [int(l.split()[1]) for l in capsys.readouterr().out.splitlines() if l.startswith("done ")]
    return rc, done


@pytest.mark.parametrize("name,cfg", [("A", TINY_A), ("B", TINY_B)])
def test_trace_run_bookkeeping(name, cfg, tiny_dirs, plain_kernels, monkeypatch, capsys, tmp_path):
    g = torch.Generator().manual_seed(21)
    reqs = {f"r{i}": torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()
            for i, n in enumerate([1, 70, 40, 90, 66])}
    tr = ru.Trace()
    ru.whole(tr, "w", reqs["r1"])
    ru.tail_decode(tr, "t", reqs["r2"], tail=5)
    ru.portions(tr, "p", reqs["r3"], sizes=[2, 3, 61, 2, 1])
    mix = {f"m{k}": v for k, v in reqs.items()}
    ru.mixed(tr, mix, seed=5, decode_tail=3)
    plain = plain_lfm2.PlainLfm2(tiny_dirs[name])
    ref = {"w": plain.logits(reqs["r1"]), "t": plain.logits(reqs["r2"]), "p": plain.logits(reqs["r3"])}
    ref.update({k: plain.logits(v) for k, v in mix.items()})
    out_dir = str(tmp_path / "out")
    rc, done = _run_in_process(monkeypatch, capsys, tiny_dirs[name], tr, out_dir, tr.peak_tokens)
    assert rc == 0 and done == list(range(len(tr.steps)))
    got = {}
    for step, rows in tr.rows.items():
        got[step] = np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(len(rows), cfg["vocab_size"])
    ok, msg = ru.compare(tr, got, ref, "float32")
    assert ok, msg


def test_trace_run_reports_out_of_pages(tiny_dirs, plain_kernels, monkeypatch, capsys, tmp_path):
    tr = ru.Trace()
    ru.whole(tr, "w", list(range(130)))
    rc, done = _run_in_process(monkeypatch, capsys, tiny_dirs["A"], tr, str(tmp_path / "o"), 128)
    assert rc == 4 and done == []
