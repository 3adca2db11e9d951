"""Trace replay: feed given token ids through the model step by step and write logits.

In the spirit of the reference's `generate --dump-logits <dir>`, which writes the raw
float32 logits of every fed token (src/main.cpp:297-307, 677-726), but nothing is sampled:
the trace says which tokens every request gets at every step and at which of them logits
are wanted.  The replay drives the same `Context.forward_batch` that generation uses.

Input, one JSON object per line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step with wanted places, `<out>/<step>.f32` gets the logits, little-endian float32
[wanted, vocab], in the order of the entries and of each entry's `want`.  After every step
`done <step>` is printed and flushed.  Requests named in `end` give their slot and pages
back after the step.

Beside the logits, `<out>/index.jsonl` gets one line per request and step: the step, the
request's id, the cache slot it holds, the positions its tokens took, and which rows of
`<step>.f32` are its wanted places (the reference writes `generation_tokens.txt` beside its
per-step files for the same purpose: to say what the files hold, src/main.cpp:322-337).
Slots that are used again by later requests show there.

The plain implementation under tests/ is not driven from here: it is test code, and the
package imports nothing from the tests.  A test that wants both runs the same trace through
it itself (tests/test_replay_gpu.py does).
"""
from __future__ import annotations

import json
import os
import sys
from typing import Dict, IO, Optional

import torch

from .batch import MiniBatch, SequenceChunk
from .context import Context


class Replayer:
    def __init__(self, context: Context, out_dir: str):
        self.ctx = context
        self.out_dir = out_dir
        os.makedirs(out_dir, exist_ok=True)
        self.slot_of: Dict[str, int] = {}
        self.index_path = os.path.join(out_dir, "index.jsonl")
        open(self.index_path, "w").close()

    def step(self, record: dict) -> Optional[torch.Tensor]:
        step_id = record["step"]
        chunks = []
        fresh = []
        try:
            for e in record.get("entries", []):
                rid = str(e["id"])
                if rid not in self.slot_of:
                    self.slot_of[rid] = self.ctx.acquire()
                    fresh.append(rid)
                chunks.append(SequenceChunk(self.slot_of[rid], [int(t) for t in e["tokens"]],
                                            [int(w) for w in e.get("want", [])]))
            logits = None
            starts = [self.ctx.length(c.slot) for c in chunks]
            if chunks:
                logits = self.ctx.forward_batch(MiniBatch(chunks))
        except Exception:
            for rid in fresh:                     # a refused step leaves no half-started request behind
                self.ctx.release(self.slot_of.pop(rid))
            raise
        if logits is not None and logits.shape[0] > 0:
            data = logits.detach().to("cpu", torch.float32).contiguous().numpy()
            path = os.path.join(self.out_dir, f"{step_id}.f32")
            with open(path + ".tmp", "wb") as f:
                f.write(data.astype("<f4", copy=False).tobytes())
            os.replace(path + ".tmp", path)
        with open(self.index_path, "a") as f:
            row = 0
            for e, c, start in zip(record.get("entries", []), chunks, starts):
                f.write(json.dumps({"step": step_id, "id": str(e["id"]), "slot": c.slot,
                                    "positions": [start, start + len(c.tokens)],
                                    "rows": list(range(row, row + len(c.want)))}) + "\n")
                row += len(c.want)
        for rid in record.get("end", []):
            rid = str(rid)
            if rid in self.slot_of:
                self.ctx.release(self.slot_of.pop(rid))
        return logits

    def run(self, lines: IO[str], out: IO[str] = sys.stdout) -> int:
        for line in lines:
            line = line.strip()
            if not line:
                continue
            record = json.loads(line)
            self.step(record)
            out.write(f"done {record['step']}\n")
            out.flush()
        return 0
