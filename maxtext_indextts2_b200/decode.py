"""Command line of the decode path (the role of ``MaxText/decode.py``): prompts in, sampled token ids out.

    python -m maxtext_indextts2_b200.decode [config.yml] key=value ... --prompt 5,17,3 [--prompt 8,2] [--max-decode 32]
    python -m maxtext_indextts2_b200.decode model_dir=/path/to/model dtype=float32 --prompt 5,17,3

With ``model_dir=`` the model class, sizes and weights come from the folder's config.json / model.safetensors
(``pyconfig.from_model_dir``: the layered designs); otherwise the keys describe a llama2 / gemma3 model with random weights or
``load_parameters_path``.  Prompts are token ids (this path has no tokenizer); they run through ``OfflineEngine`` -- continuous
batching over ``per_device_batch_size`` slots, the configured ``decode_sampling_strategy`` -- and one JSON line per prompt is
printed: {"prompt": i, "tokens": [...]}.
"""

from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
  ap = argparse.ArgumentParser(prog="decode", description=__doc__.split("\n")[0])
  ap.add_argument("config", nargs="*", help="[config.yml] key=value ...")
  ap.add_argument("--prompt", action="append", default=[], help="comma-separated token ids; may be given several times")
  ap.add_argument("--max-decode", type=int, default=16)
  ap.add_argument("--eos", type=int, action="append", default=[])
  a = ap.parse_args(argv)

  from . import _lib, offline_engine, pyconfig

  _lib.build()
  pairs = dict(kv.split("=", 1) for kv in a.config if "=" in kv)
  prompts = [[int(t) for t in p.split(",") if t.strip()] for p in a.prompt] or [[1, 2, 3]]
  if "model_dir" in pairs:
    model_dir = pairs.pop("model_dir")
    longest = max(len(p) for p in prompts) + a.max_decode + 1
    typed = {k: pyconfig._parse_like(pyconfig._load_yaml(pyconfig.BASE_YML)[k], v, k) for k, v in pairs.items()}
    typed.setdefault("per_device_batch_size", min(4, len(prompts)))
    typed.setdefault("max_target_length", longest)
    tpp = int(typed.setdefault("pagedattn_tokens_per_page", 64))
    typed.setdefault("pagedattn_num_pages", int(typed["per_device_batch_size"]) * ((int(typed["max_target_length"]) + tpp - 1) // tpp) + 1)
    config = pyconfig.from_model_dir(model_dir, **typed)
    params = None
  else:
    config = pyconfig.initialize([sys.argv[0]] + a.config)
    params = None
  engine = offline_engine.OfflineEngine(config, params=params, eos_ids=a.eos)
  for out in engine.batch_inference(prompts, max_decode_length=a.max_decode):
    print(json.dumps({"prompt": out.index, "tokens": out.token_ids.tolist()}), flush=True)
  return 0


if __name__ == "__main__":
  sys.exit(main())
