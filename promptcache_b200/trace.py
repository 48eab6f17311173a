"""Trace replay: feed given token ids through a model step by step and write the logits that are asked for.

    python -m promptcache_b200.trace --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N   (bin/trace_run)

reads one JSON object per line from standard input,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}

runs the entries of a step as ONE batch through the `BatchEngine` (a request id seen for the first time starts at its
first token, a known one continues from the state its earlier steps left; `end` gives requests' slots back), writes
DIR/<step>.f32 (little-endian float32 [wanted, vocab], in the order of the entries and of `want`) when something was
wanted, and prints `done <step>`.  Nothing is sampled.  The model class is chosen by config.json's "architecture".
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder the logits files are written to")
    ap.add_argument("--max-tokens", type=int, default=None, help="most tokens live requests hold at any time (sizes the slot pool)")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    import torch
    from .batch_engine import BatchEngine
    from .model import load_model
    if not torch.cuda.is_available():
        print("trace_run: no CUDA device (this framework has no CPU path)", file=sys.stderr)
        return 2
    torch.cuda.set_device(torch.device(args.device))
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    model = load_model(args.model, device=args.device, dtype=dtype)
    engine = BatchEngine(model, max_tokens=args.max_tokens)
    os.makedirs(args.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        req = json.loads(line)
        entries = [(e["id"], e["tokens"], e.get("want", [])) for e in req.get("entries", [])]
        logits = engine.step(entries, req.get("end", []))
        if logits.shape[0] > 0:
            data = logits.to(torch.float32).contiguous().cpu().numpy().astype("<f4", copy=False).tobytes()
            tmp = os.path.join(args.out, f".{req['step']}.f32.part")
            with open(tmp, "wb") as fh:
                fh.write(data)
            os.replace(tmp, os.path.join(args.out, f"{req['step']}.f32"))
        else:
            torch.cuda.synchronize()
        print(f"done {req['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
