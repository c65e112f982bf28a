"""Command line of the language-model engines:  python -m leopard_b200 <command>

  models                                   the architectures the registry can load
  generate --model DIR --prompt 1,2,3 ...  continue token-id prompts through the scheduler (greedy unless --temperature)
  trace --model DIR --out DIR              replay a step trace from standard input and write the logits asked for

`trace` reads one JSON object per line: {"step": n, "entries": [{"id", "tokens", "want"}], "end": [ids]}.  Every entry brings a
request's next tokens; all entries of a step run as one batch through the engine's step function, from the cache and state the
earlier steps left.  For a step that wants logits it writes <out>/<step>.f32 (little-endian fp32 [wanted, vocab], in the order of the
entries and of their `want` lists), then prints `done <step>`.  Requests named in `end` give their cache pages and state slot back.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional


def _load(args):
    from . import registry
    return registry.load_model(args.model, dtype=args.dtype, max_tokens=args.max_tokens)


def cmd_models(args) -> int:
    from . import registry
    print("\n".join(registry.architectures()))
    return 0


def cmd_generate(args) -> int:
    from .sampling import SamplingParams
    from .scheduler import generate
    eng = _load(args)
    prompts = [[int(t) for t in p.split(",") if t.strip()] for p in args.prompt]
    outs = generate(eng, prompts, max_new_tokens=args.max_new_tokens, eos=set(args.eos or ()),
                    sampling=SamplingParams(temperature=args.temperature, top_k=args.top_k, seed=args.seed))
    for p, o in zip(prompts, outs):
        print(json.dumps({"prompt": p, "output": o}))
    return 0


def cmd_trace(args) -> int:
    from .seqlm import StepEntry
    eng = _load(args)
    if not hasattr(eng, "step"):
        print("this architecture has no step engine", file=sys.stderr)
        return 2
    os.makedirs(args.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = [StepEntry(e["id"], e["tokens"], e.get("want") or []) for e in step["entries"]]
        logits = eng.step(entries)
        if logits is not None:
            tmp = os.path.join(args.out, f".{step['step']}.part")
            logits.float().cpu().numpy().astype("<f4").tofile(tmp)
            os.replace(tmp, os.path.join(args.out, f"{step['step']}.f32"))
        for key in step.get("end") or []:
            eng.finish(key)
        sys.stdout.write(f"done {step['step']}\n")
        sys.stdout.flush()
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="leopard_b200", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)
    sub.add_parser("models").set_defaults(fn=cmd_models)
    for name, fn in (("generate", cmd_generate), ("trace", cmd_trace)):
        p = sub.add_parser(name)
        p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
        p.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
        p.add_argument("--max-tokens", type=int, default=4096, help="tokens that live requests hold at most (first cache size)")
        p.set_defaults(fn=fn)
        if name == "generate":
            p.add_argument("--prompt", action="append", required=True, help="comma-separated token ids; repeat for a batch")
            p.add_argument("--max-new-tokens", type=int, default=16)
            p.add_argument("--eos", type=int, action="append")
            p.add_argument("--temperature", type=float, default=0.0)
            p.add_argument("--top-k", type=int, default=0)
            p.add_argument("--seed", type=int)
        else:
            p.add_argument("--out", required=True)
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
