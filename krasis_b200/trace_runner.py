"""Replay a trace of steps through the serving path and write the requested logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--max-requests 4]

Reads one JSON object per line from standard input,
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}
runs every step's entries as one batch through `Scheduler.step` (the model, cache pool, state slots and kernels of the generation
path), writes DIR/<step>.f32 ([wanted, vocab] little-endian float32) when a step wants logits, releases the requests named in
"end", and prints "done <step>".  Nothing is sampled.  Exit code 0 at end of input."""
import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, required=True)
    ap.add_argument("--max-requests", type=int, default=4)
    ap.add_argument("--device", type=int, default=0)
    a = ap.parse_args(argv)

    import torch
    from .registry import load_model
    from .scheduler import Scheduler

    dtype = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    model = load_model(a.model, dtype=dtype, device=a.device)
    if not hasattr(model, "forward_step"):
        print(f"{type(model).__name__} has no step interface for trace replay", file=sys.stderr)
        return 3
    sched = Scheduler(model, max_tokens=a.max_tokens, max_requests=a.max_requests)
    os.makedirs(a.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        msg = json.loads(line)
        logits = sched.step([(e["id"], e["tokens"], e.get("want", [])) for e in msg.get("entries", [])])
        if logits is not None:
            data = logits.to(torch.float32).contiguous().cpu().numpy().astype("<f4")
            tmp = os.path.join(a.out, f".{msg['step']}.part")
            with open(tmp, "wb") as f:
                f.write(data.tobytes())
            os.replace(tmp, os.path.join(a.out, f"{msg['step']}.f32"))
        else:
            torch.cuda.synchronize()
        for rid in msg.get("end", []):
            if rid in sched.live:
                sched.finish(rid)
        sys.stdout.write(f"done {msg['step']}\n")
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
