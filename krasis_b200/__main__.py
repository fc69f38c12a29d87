"""Command line of the serving path.

    python -m krasis_b200 generate --model DIR --prompt-ids 5,17,3 [--prompt-ids ...] [--max-new-tokens 32] [--dtype bfloat16]
                                   [--temperature 0 --top-k 0 --top-p 1 --seed 0] [--max-tokens 8192] [--step-tokens 512]
    python -m krasis_b200 trace    --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N        (same as bin/trace_run)

`generate` loads the checkpoint through the model registry (config.json decides the class), runs continuous batching over the
given prompts and prints one JSON line per prompt with the generated token ids.  Token ids in, token ids out: tokenisers are not
part of this package."""
import argparse
import json
import sys


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if argv and argv[0] == "trace":
        from .trace_runner import main as trace_main
        return trace_main(argv[1:])
    ap = argparse.ArgumentParser(prog="python -m krasis_b200", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("command", choices=["generate"])
    ap.add_argument("--model", required=True)
    ap.add_argument("--prompt-ids", action="append", required=True, help="comma-separated token ids; repeat for several prompts")
    ap.add_argument("--max-new-tokens", type=int, default=32)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=None)
    ap.add_argument("--eos", type=int, default=None)
    ap.add_argument("--max-tokens", type=int, default=8192, help="tokens the cache pool holds")
    ap.add_argument("--max-requests", type=int, default=4)
    ap.add_argument("--step-tokens", type=int, default=512, help="token budget of one step (prompt portions + decoded tokens)")
    a = ap.parse_args(argv)

    import torch
    from .registry import load_model
    from .sampling import SamplingParams
    from .scheduler import Scheduler
    model = load_model(a.model, dtype=torch.bfloat16 if a.dtype == "bfloat16" else torch.float32)
    if not hasattr(model, "forward_step"):
        print(f"{type(model).__name__} has no step interface for generation", file=sys.stderr)
        return 3
    prompts = [[int(t) for t in p.split(",") if t.strip()] for p in a.prompt_ids]
    sched = Scheduler(model, max_tokens=a.max_tokens, max_requests=a.max_requests, cuda_graphs=True)
    outs = sched.generate(prompts, a.max_new_tokens, SamplingParams(a.temperature, a.top_k, a.top_p, a.seed), step_tokens=a.step_tokens,
                          eos=a.eos)
    for p, o in zip(prompts, outs):
        print(json.dumps({"prompt_tokens": len(p), "generated": o}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
