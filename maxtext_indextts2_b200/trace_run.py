"""Replay a trace of batched steps through the engine and write the logits it asks for.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

`--model` is a folder with config.json and model.safetensors; the model class is chosen by config.json
(``pyconfig.from_model_dir``).  Standard input carries one JSON object per line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

Every entry gives a request's next tokens and the places among them whose logits are wanted; all entries of a step run as ONE
ragged batch of the engine (``MaxEngine.step``): portions of prompts beside single decoded tokens.  A request takes a decode slot
(page group) at its first entry and gives it and its pages back when it is listed in "end".  For a step that wants something
the logits are written to ``<out>/<step>.f32`` ([wanted, vocab] little-endian float32, in the order of the entries); after every
step the line ``done <step>`` is printed.  The cache pool holds `--max-tokens` tokens in pages of 64 for at most four live
requests.  Nothing is sampled.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

SLOTS = 4
TOKENS_PER_PAGE = 64


def main(argv=None) -> int:
  ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n")[0])
  ap.add_argument("--model", required=True)
  ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
  ap.add_argument("--out", required=True)
  ap.add_argument("--max-tokens", type=int, required=True)
  a = ap.parse_args(argv)

  from . import _lib

  _lib.build()  # compiles on the first call in a fresh checkout, a no-op afterwards
  import numpy as np
  import torch

  from . import maxengine, pyconfig

  pages = (a.max_tokens + TOKENS_PER_PAGE - 1) // TOKENS_PER_PAGE
  config = pyconfig.from_model_dir(
      a.model, dtype=a.dtype, per_device_batch_size=SLOTS, max_target_length=pages * TOKENS_PER_PAGE + 1,
      pagedattn_tokens_per_page=TOKENS_PER_PAGE, pagedattn_num_pages=pages + 1,  # page 0 is never handed out
      pagedattn_max_pages_per_group=pages + 1)
  torch.cuda.set_device(0)
  engine = maxengine.MaxEngine(config)
  engine.load_params()
  engine.init_decode_state()
  os.makedirs(a.out, exist_ok=True)
  slot_of, free = {}, list(range(SLOTS))[::-1]
  for line in sys.stdin:
    line = line.strip()
    if not line:
      continue
    msg = json.loads(line)
    entries = []
    for e in msg.get("entries", []):
      rid = e["id"]
      if rid not in slot_of:
        if not free:
          raise RuntimeError(f"request {rid!r}: all {SLOTS} slots are taken")
        slot_of[rid] = free.pop()
      entries.append((slot_of[rid], e["tokens"], e.get("want", [])))
    logits = engine.step(entries)
    if logits.shape[0]:
      host = logits.cpu().numpy().astype("<f4", copy=False)
      tmp = os.path.join(a.out, f".{msg['step']}.f32.part")
      with open(tmp, "wb") as f:
        f.write(np.ascontiguousarray(host).tobytes())
      os.replace(tmp, os.path.join(a.out, f"{msg['step']}.f32"))
    for rid in msg.get("end", []):
      if rid in slot_of:
        slot = slot_of.pop(rid)
        engine.release_pages(slot)
        free.append(slot)
    sys.stdout.write(f"done {msg['step']}\n")
    sys.stdout.flush()
  return 0


if __name__ == "__main__":
  sys.exit(main())
