"""Command line: ``python -m vapi_b200 [--config vapi.toml] [options] --prompt-ids 1,2,3``.

In the reference's manner the configuration is a TOML file named by ``--config`` / ``-c``
(or ``$VAPI_CONFIG``, or ``./vapi.toml``), and an argument that is not known is an error
that names it (crates/vapi-core/src/cli.rs:26-56, crates/vapi-worker/src/main.rs:24-52).
Where the reference's worker takes its jobs from a queue, this program takes prompts as
token ids from flags or from standard input (one JSON list per line) and prints one JSON
object per completion.  Every ``[model]`` / ``[worker]`` / ``[cache]`` key can also be given
as a flag of the same name, which wins over the file.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import List, Optional


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="vapi_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter, allow_abbrev=False)
    ap.add_argument("-c", "--config", help="TOML file with [model], [worker], [cache]")
    g = ap.add_argument_group("[model]")
    g.add_argument("--path", "--model", dest="path", help="model folder (config.json + safetensors)")
    g.add_argument("--dtype", choices=["auto", "bf16", "bfloat16", "f32", "float32"])
    g.add_argument("--max-context", type=int)
    g.add_argument("--kv-cache-fraction", type=float)
    g.add_argument("--num-blocks", type=int)
    g.add_argument("--cuda-graphs", dest="cuda_graphs", action="store_true", default=None)
    g.add_argument("--no-cuda-graphs", dest="cuda_graphs", action="store_false")
    g.add_argument("--random-weights", type=int, metavar="SEED",
                   help="draw random weights for --config-json instead of loading a folder")
    g.add_argument("--config-json", help="a config.json to use with --random-weights")
    g = ap.add_argument_group("[worker]")
    g.add_argument("--max-concurrent-seqs", type=int)
    g.add_argument("--max-batched-tokens", type=int)
    g.add_argument("--prefill-chunk-tokens", type=int)
    g.add_argument("--max-step-failures", type=int)
    g = ap.add_argument_group("[cache]")
    g.add_argument("--watermark", type=float)
    g = ap.add_argument_group("sampling")
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--top-k", type=int)
    g.add_argument("--min-p", type=float, default=0.0)
    g.add_argument("--repetition-penalty", type=float, default=1.0)
    g.add_argument("--frequency-penalty", type=float, default=0.0)
    g.add_argument("--presence-penalty", type=float, default=0.0)
    g.add_argument("--max-tokens", type=int, default=256)
    g.add_argument("--seed", type=int)
    g.add_argument("--n", type=int, default=1, help="completions per prompt")
    g.add_argument("--logprobs", type=int, help="report log-probabilities: the chosen token's and this many top ones")
    g.add_argument("--stop-token-ids", default="", help="comma-separated token ids")
    g = ap.add_argument_group("prompts")
    g.add_argument("--prompt-ids", action="append", default=[], metavar="ID,ID,...",
                   help="a prompt as comma-separated token ids (repeatable); without it, "
                        "JSON lists are read from standard input, one per line")
    g.add_argument("--stats", action="store_true", help="print engine statistics to stderr at the end")
    return ap


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    from .config.runtime import RuntimeConfig, RuntimeConfigError
    try:
        cfg = RuntimeConfig.load(args.config)
    except RuntimeConfigError as e:
        print(f"vapi_b200: {e}", file=sys.stderr)
        return 2
    for sec, keys in (("model", ("path", "dtype", "max_context", "kv_cache_fraction", "num_blocks", "cuda_graphs")),
                      ("worker", ("max_concurrent_seqs", "max_batched_tokens", "prefill_chunk_tokens", "max_step_failures")),
                      ("cache", ("watermark",))):
        for k in keys:
            v = getattr(args, k)
            if v is not None:
                setattr(getattr(cfg, sec), k, v)
    try:
        cfg.validate()
    except RuntimeConfigError as e:
        print(f"vapi_b200: {e}", file=sys.stderr)
        return 2
    prompts = [[int(t) for t in s.split(",") if t.strip()] for s in args.prompt_ids]
    if not prompts:
        for line in sys.stdin:
            line = line.strip()
            if line:
                prompts.append([int(t) for t in json.loads(line)])
    if not prompts:
        print("vapi_b200: no prompts given", file=sys.stderr)
        return 2

    from .api import LLM
    from .sampling.params import SamplingParams
    overrides = {}
    if args.random_weights is not None:
        if not args.config_json:
            print("vapi_b200: --random-weights needs --config-json", file=sys.stderr)
            return 2
        with open(args.config_json) as f:
            overrides = dict(random_weights=args.random_weights, config_json=json.load(f), model=None)
    elif not cfg.model.path:
        print("vapi_b200: no model: give [model] path, --path, or --random-weights with --config-json", file=sys.stderr)
        return 2
    llm = LLM.from_config(cfg, **overrides)
    params = SamplingParams(
        temperature=args.temperature, top_p=args.top_p, top_k=args.top_k, min_p=args.min_p,
        repetition_penalty=args.repetition_penalty, frequency_penalty=args.frequency_penalty,
        presence_penalty=args.presence_penalty, max_tokens=args.max_tokens, seed=args.seed, n=args.n,
        logprobs=args.logprobs,
        stop_token_ids=tuple(int(t) for t in args.stop_token_ids.split(",") if t.strip()))
    from .engine.scheduler import AdmitError
    try:
        completions = llm.generate(prompts, params)
    except (AdmitError, ValueError) as e:       # a prompt or a sampling parameter that cannot be served
        print(f"vapi_b200: {e}", file=sys.stderr)
        return 2
    for c in completions:
        rec = {"request": c.request_id, "prompt_tokens": c.prompt_tokens, "tokens": c.tokens,
               "finish_reason": c.finish_reason}
        if params.n > 1:
            rec["index"] = c.index
        if c.logprobs is not None:
            rec["logprobs"] = [{"token": lp.token, "logprob": lp.logprob, "top": lp.top} for lp in c.logprobs]
        print(json.dumps(rec), flush=True)
    if args.stats:
        print(json.dumps(llm.engine.stats.__dict__), file=sys.stderr)
    return 0
