"""Trace replay: feed given token ids through a model step by step and write the logits of the wanted places.

Steps arrive on standard input, one JSON object per line:
    {"step": n, "entries": [{"id": "a", "tokens": [...], "want": [...]}], "end": ["a", ...]}
Each entry brings a request's next tokens; `want` are offsets among them.  The rows go through the engine's step
function against the caches and states earlier steps left; requests named in `end` give their slots back.  For a step
with wanted places, <out>/<n>.f32 gets their logits ([wanted, vocab] little-endian float32, in the order of the entries
and of `want`); after every step a line "done <n>" is printed.  Nothing is sampled.
"""
import json
import os
import sys

import numpy as np


def replay(model, lines, out_dir, emit=print):
    from .engine import Engine
    eng = Engine(model)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = []
        for e in step.get("entries", []):
            if eng.open(e["id"]) is None:
                raise RuntimeError("no free slot for request %r" % (e["id"],))
            entries.append((e["id"], e["tokens"], e.get("want", [])))
        res = eng.forward_step([x for x in entries if len(x[1])], want_logits=True) if entries else {}
        rows = []
        for rid, tokens, want in entries:
            if len(want):
                logits = res[rid][1]
                order = {w: i for i, w in enumerate(sorted(set(want)))}
                rows += [logits[order[w]] for w in want]
        if rows:
            np.stack(rows).astype("<f4").tofile(os.path.join(out_dir, "%d.f32" % step["step"]))
        for rid in step.get("end", []):
            eng.close(rid)
        emit("done %d" % step["step"])
        sys.stdout.flush()
