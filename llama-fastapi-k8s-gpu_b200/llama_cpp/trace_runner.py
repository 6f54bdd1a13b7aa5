"""Replay a trace of token steps through an engine and write the logits (no sampling).

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input carries one JSON object per line,
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}
Each entry brings the next tokens of request `id` (admitted at its first entry) and the places among them whose
logits are asked for; all entries of a line run as ONE ragged engine step, prompt portions beside single decoded
tokens. For a step with wanted places the logits go to <out>/<step>.f32 ([wanted, vocab] little-endian float32, in
entry order); after every step a line `done <step>` is printed. Requests listed in `end` give their pages and state
slot back. The page pool is sized for --max-tokens (each live request rounded up to whole pages) and four slots.

This drives the same objects the serving path uses: `models.open_model` / `open_engine` (registry), the engine's
`step`, `SequenceSlots` + `PageAllocator` (pages and recurrent-state slots).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np

MAX_LIVE = 4


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors, or a GGUF file")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True, help="most tokens live requests hold at any time")
    ap.add_argument("--device", type=int, default=0)
    a = ap.parse_args(argv)

    import build as native_build          # compiles the CUDA library in-tree when it is missing or stale
    native_build.build()
    from . import models
    from .kv_pages import SequenceSlots

    src = models.open_model(a.model)
    if src.family.source != "folder":
        print("trace_run: this model family is served by the request scheduler only (no ragged step)", file=sys.stderr)
        return 2
    block = 64
    # every live request may round up to a whole page
    pool_tokens = a.max_tokens + MAX_LIVE * block
    eng = models.open_engine(src, n_ctx=max(a.max_tokens, block), max_seqs=MAX_LIVE, device=a.device, kv_block_tokens=block,
                             dtype=a.dtype, kv_tokens=pool_tokens)
    seqs = SequenceSlots(eng)
    os.makedirs(a.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        msg = json.loads(line)
        entries, want = [], []
        for en in msg.get("entries", []):
            key, toks = en["id"], [int(t) for t in en["tokens"]]
            if not toks:
                continue
            if key not in seqs:
                seqs.open(key)
            slot = seqs.extend(key, len(toks))
            entries.append((slot, toks))
            want.append([int(w) for w in en.get("want", [])])
        if entries:
            logits, _ = eng.step(entries, want=want)
            if logits.shape[0]:
                tmp = os.path.join(a.out, f".{msg['step']}.tmp")
                np.ascontiguousarray(logits, dtype="<f4").tofile(tmp)
                os.replace(tmp, os.path.join(a.out, f"{msg['step']}.f32"))
        for key in msg.get("end", []):
            if key in seqs:
                seqs.close(key)
        sys.stdout.write(f"done {msg['step']}\n")
        sys.stdout.flush()
    eng.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
