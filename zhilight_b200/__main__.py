"""Command line of the framework.

    python -m zhilight_b200 build
    python -m zhilight_b200 generate --model DIR [--dtype bfloat16] --prompt-ids 1,2,3 [--prompt-ids ...]
                                     [--max-new-tokens N] [--temperature T --top-k K --top-p P --seed S]
    python -m zhilight_b200 trace --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N   (steps on stdin)
"""
import argparse
import json
import os
import sys


def _build(family=None):
    """The whole library, or -- in a checkout without it -- only what `family` needs."""
    from . import _lib, build
    path = build.build(family=family)
    if path != build.LIB_PATH:
        _lib.use(path)
    return path


def main(argv=None):
    ap = argparse.ArgumentParser(prog="zhilight_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("build")
    g = sub.add_parser("generate")
    g.add_argument("--model", required=True)
    g.add_argument("--dtype", default="bfloat16")
    g.add_argument("--prompt-ids", action="append", required=True, help="comma-separated token ids; repeat for a batch")
    g.add_argument("--max-new-tokens", type=int, default=16)
    g.add_argument("--max-batch", type=int, default=8)
    g.add_argument("--max-seq", type=int, default=4096)
    g.add_argument("--max-step-tokens", type=int, default=512)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--seed", type=int, default=0)
    t = sub.add_parser("trace")
    t.add_argument("--model", required=True)
    t.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    t.add_argument("--out", required=True)
    t.add_argument("--max-tokens", type=int, default=4096)
    t.add_argument("--max-step-tokens", type=int, default=512)
    a = ap.parse_args(argv)

    if a.cmd == "build":
        print(_build())
        return 0
    from . import registry
    if a.cmd == "trace":
        with open(os.path.join(a.model, "config.json")) as f:
            config = json.load(f)
        if a.dtype not in registry.supported_dtypes(config):
            sys.stderr.write("%s does not run in %s\n" % (registry.architecture_of(config), a.dtype))
            return 3
    with open(os.path.join(a.model, "config.json")) as f:
        _build(family=str(registry.architecture_of(json.load(f))))
    if a.cmd == "generate":
        from .engine import Engine, SamplingParams
        prompts = [[int(x) for x in p.split(",") if x.strip()] for p in a.prompt_ids]
        model = registry.load_model(a.model, a.dtype, max_batch=min(a.max_batch, max(1, len(prompts))), max_seq=a.max_seq,
                                    max_step_tokens=a.max_step_tokens)
        sp = [SamplingParams(a.temperature, a.top_k, a.top_p, a.seed + i) for i in range(len(prompts))]
        for p, out in zip(prompts, Engine(model).generate(prompts, a.max_new_tokens, sp)):
            print(json.dumps({"prompt": p, "output": out}))
        return 0
    from . import trace
    os.makedirs(a.out, exist_ok=True)
    model = registry.load_model(a.model, a.dtype, max_batch=4, max_seq=max(a.max_tokens, 1),
                                max_step_tokens=a.max_step_tokens)
    trace.replay(model, sys.stdin, a.out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
