"""Trace replay: feeds given token ids through a model step by step and writes the logits of chosen places.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR [--max-tokens N]

Standard input carries one JSON object per line,
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}
`entries` brings each request's next tokens (a prompt portion of any length, or one token) and the places among them
whose logits are wanted; `end` lists the requests whose state and pages go back to the pool after the step. For a step
with wanted places the fp32 logits [wanted, vocab] go to DIR/<step>.f32 (little-endian, entry order); after every step a
line `done <step>` is printed. Nothing is sampled. The model class comes from config.json through the registry and the
step is the engine's own scheduler step (`forward_step`): the same kernels, state slots and pages that `generate` uses."""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="directory with config.json and *.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="directory that receives <step>.f32")
    ap.add_argument("--max-tokens", type=int, default=0, help="most tokens live requests hold at any time (sizes the pools)")
    a = ap.parse_args(argv)

    import torch

    from .registry import architecture_of, model_class

    with open(os.path.join(a.model, "config.json")) as f:
        cls = model_class(architecture_of(json.load(f)))
    if not hasattr(cls, "forward_step"):
        print(f"{cls.__name__} has no teacher-forced step", file=sys.stderr)
        return 3
    model = cls.from_pretrained(a.model, torch_dtype=a.dtype, device_map="cuda", max_tokens=a.max_tokens)
    os.makedirs(a.out, exist_ok=True)
    live = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries, want = [], []
        for e in step.get("entries", []):
            cache = live.get(e["id"])
            if cache is None:
                cache = live[e["id"]] = model.new_cache()
            entries.append((cache, e["tokens"]))
            want.append(e.get("want", []))
        if entries:
            logits = model.forward_step(entries, want)
            if logits is not None and logits.shape[0]:
                data = logits.to(torch.float32).cpu().contiguous().numpy().astype("<f4", copy=False).tobytes()
                tmp = os.path.join(a.out, f".{step['step']}.part")
                with open(tmp, "wb") as f:
                    f.write(data)
                os.replace(tmp, os.path.join(a.out, f"{step['step']}.f32"))
            else:
                torch.cuda.synchronize()
        for rid in step.get("end", []):
            cache = live.pop(rid, None)
            if cache is not None:
                cache.release()
        sys.stdout.write(f"done {step['step']}\n")
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
