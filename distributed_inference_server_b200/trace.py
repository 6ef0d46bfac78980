"""Trace replay: feed given token ids through a model step by step and write the logits at the asked positions.

    python -m distributed_inference_server_b200.trace --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input carries one JSON object per line,
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
`entries` lists, per request, its next tokens and the offsets among them whose logits are wanted; `end` the requests that
are finished after the step.  All entries of a step run as ONE pass of the engine (dis_engine_step): portions of prompts
beside single tokens, from the cache pages and state slots that earlier steps left.  For a step in which something is
wanted, <out>/<step>.f32 receives the logits [wanted, vocab] as little-endian float32, in the order of the entries and of
`want`; after every step `done <step>` is printed.  Nothing is sampled into the sequences: the tokens are the caller's.

This module has no forward pass, cache or loader of its own; it drives models.load_model and the Engine wrapper, i.e. the
same sequences, page allocator, step planner and kernels that generation uses.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, required=True)
    ap.add_argument("--max-requests", type=int, default=4, help="state slots (requests live at one time)")
    ap.add_argument("--page-size", type=int, default=64)
    a = ap.parse_args(argv)

    from . import build
    build.build()  # incremental: compiles at the first call in a fresh checkout, a no-op afterwards
    from . import models
    from .worker import InferenceParams

    page = a.page_size
    pool = (max(a.max_tokens, 1) + page - 1) // page * page
    family, _ = models.read_config(a.model)
    if family != "stack" and a.dtype == "float32":
        sys.stderr.write("trace: this model family computes in bfloat16 only\n")
        return 3
    eng = models.load_model(a.model, dtype=a.dtype, max_batch=a.max_requests, max_tokens=pool, page_size=page,
                            max_step_tokens=pool, max_logit_rows=pool + a.max_requests, max_ctx=pool + page)
    os.makedirs(a.out, exist_ok=True)
    params = InferenceParams(max_tokens=1 << 30, temperature=0.0)
    slots = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        st = json.loads(line)
        listed, wants = [], []
        for en in st.get("entries", []):
            toks, want = [int(t) for t in en["tokens"]], [int(w) for w in en.get("want", [])]
            if not toks:
                continue
            order = sorted(set(want))
            rid = en["id"]
            if rid not in slots:
                slots[rid] = eng.seq_add(toks, params)
                eng.seq_probe(slots[rid], order)
            else:
                eng.seq_extend(slots[rid], toks, order)
            listed.append(slots[rid])
            wants.append((want, order, len(toks)))
        rows = []
        if listed:
            left = {s: n for s, (_, _, n) in zip(listed, wants)}
            got = {s: [] for s in listed}
            while left:  # one pass unless the step is larger than the engine's pass capacity
                run = [s for s in listed if s in left]
                _, _, prod = eng.step(run)
                n_rows = eng.last_logit_rows()
                lg = eng.last_logits(n_rows) if n_rows else np.zeros((0, eng.vocab), np.float32)
                # rows: per listed sequence its probed positions in ascending order, then its sampled row if the pass
                # reached the end of its tokens
                at = 0
                for s, p in zip(run, prod):
                    k = len(wants[listed.index(s)][1]) - len(got[s])
                    if not p:  # more of this portion to come: every row so far is a probe
                        k_now = n_rows - at if s == run[-1] else None
                        if k_now is None:
                            raise RuntimeError("trace: a pass split a portion that was not the last listed")
                        got[s].extend(lg[at:at + k_now])
                        at += k_now
                        continue
                    got[s].extend(lg[at:at + k])
                    at += k + 1
                    del left[s]
            for s, (want, order, _) in zip(listed, wants):
                index = {w: i for i, w in enumerate(order)}
                rows.extend(got[s][index[w]] for w in want)
        if rows:
            np.stack(rows).astype("<f4").tofile(os.path.join(a.out, f"{st['step']}.f32"))
        for rid in st.get("end", []):
            if rid in slots:
                eng.seq_remove(slots.pop(rid))
        sys.stdout.write(f"done {st['step']}\n")
        sys.stdout.flush()
    eng.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
