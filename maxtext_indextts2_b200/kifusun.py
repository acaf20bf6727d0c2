"""The Kifusun design: a decoder whose layers are listed one by one in the model's config.json.

A layer is ``x += g1 * unit(mixer(x))`` then (if it has one) ``x += g2 * unit(ff(x))``: the sublayers read the residual stream
itself and the normalisation (``unit(y) = y / sqrt(mean(y^2) + eps)``, one gain per norm) sits on their OUTPUT.  The mixer
"attention" is a sliding-window attention without softmax and without rotation (csrc/window_attention.cuh): biased q/k/v
projections, per-head RMS norm of q and k, ``cap * tanh(scale * q.k / cap)`` plus a learned bias by (bucketed) distance, a
sigmoid per key with a per-head bias, mixing of the heads' weights by an [H, H] matrix, and values that every value-mixing layer
but the first blends with the first one's values of the same token.  The feed-forward is ``down(gelu_tanh(gate x) * up x)``.

This module is the design's entry in the framework: config.json -> config keys (`config_keys`, used by
``pyconfig.from_model_dir``), checks of the layer list, safetensors names -> the layer descriptors of the layered engine
(`layer_plan`), and random weights of any size for benchmarks (`random_tensors`).  No arithmetic of the model happens here.
"""

from __future__ import annotations

import math
from typing import Any, Dict, List

import numpy as np
import torch

MIXERS = ("attention",)
FF_KINDS = ("dense",)


def config_keys(model: dict) -> dict:
  """config.json of a Kifusun model -> keys of configs/base.yml."""
  layers = model["layers"]
  first = layers[0]["mixer"]
  ffs = [int(l["mlp"]["ff"]) for l in layers if l.get("mlp")]
  return dict(
      base_emb_dim=int(model["width"]),
      vocab_size=int(model["vocab"]),
      base_num_decoder_layers=len(layers),
      global_parameter_scale=1,
      normalization_layer_epsilon=float(model["norm"]["eps"]),
      embedding_scale=float(model["embedding"]["scale"]),
      layer_specs=layers,
      # (the homogeneous keys describe the first layer; the engine reads layer_specs)
      base_num_query_heads=int(first["heads"]),
      base_num_kv_heads=int(first["kv_heads"]),
      head_dim=int(first["dim"]),
      base_mlp_dim=max(ffs) if ffs else 0,
  )


def validate_layer_specs(specs: List[dict]) -> None:
  shared = None
  for i, l in enumerate(specs):
    if l.get("type") not in MIXERS:
      raise ValueError(f"layer {i}: mixer type {l.get('type')!r}; this design has {MIXERS}")
    m = l["mixer"]
    for k in ("heads", "kv_heads", "dim", "vdim", "scale", "bias_max"):
      if k not in m:
        raise ValueError(f"layer {i}: mixer.{k} is missing")
    if int(m["heads"]) % int(m["kv_heads"]):
      raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
    if int(m["mask"]["size"]) < 1:
      raise ValueError(f"layer {i}: mask.size must be positive")
    if m.get("v_mix"):
      size = (int(m["kv_heads"]), int(m["vdim"]))
      if shared is not None and size != shared:
        raise ValueError(f"layer {i}: value mixing needs (kv_heads, vdim) = {shared} as in the first mixing layer")
      shared = size if shared is None else shared
    ff = l.get("mlp")
    if ff is not None and ff.get("kind", "dense") not in FF_KINDS:
      raise ValueError(f"layer {i}: feed-forward kind {ff.get('kind')!r}; this design has {FF_KINDS}")


def distance_bucket_table(window: int, rows: int, far: float) -> np.ndarray:
  """bucket(n) for n in [0, window): n itself below rows // 2, then rows - rows // 2 logarithmic steps up to the distance `far`,
  capped at the last row.  Evaluated in float32, like everything about positions in this design."""
  half = rows // 2
  n = np.arange(window, dtype=np.int64)
  out = n.copy()
  big = n >= half
  if big.any():
    ratio = np.log(n[big].astype(np.float32) / np.float32(half)) / np.float32(math.log(far / half))
    out[big] = np.minimum(rows - 1, half + np.floor(ratio * np.float32(rows - half)).astype(np.int64))
  return out


def layer_plan(config, tensors: Dict[str, torch.Tensor], i: int, first_mix: int) -> Dict[str, Any]:
  """What layer i hands to the layered engine: sizes and scalars (python numbers) and host tensors.  Matrices keep their stored
  dtype; the engine casts them to its matmul dtype.  `first_mix`: index of the first value-mixing layer (-1: none)."""
  spec = config.layer_specs[i]
  m, p = spec["mixer"], f"l{i}.mix."
  H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
  window = int(m["mask"]["size"])
  t = tensors
  f32 = lambda name: t[name].to(torch.float32)
  rel = f32(p + "rel")  # [rows, H]
  if rel.shape[1] != H:
    raise ValueError(f"{p}rel has {rel.shape[1]} columns for {H} heads")
  buckets = torch.from_numpy(distance_bucket_table(window, int(rel.shape[0]), float(m["bias_max"])))
  plan: Dict[str, Any] = dict(
      mixer="window_sigmoid", heads=H, kv_heads=G, dim=d, vdim=dv, window=window,
      scale=float(m["scale"]), softcap=float(m.get("softcap") or 0.0),
      value_mix=0, value_lambda=0.0,
      gain1=float(f32(f"l{i}.norm1")), gain2=0.0, ff=0,
      wqkv=torch.cat([t[p + "q"], t[p + "k"], t[p + "v"]], dim=0),
      bqkv=torch.cat([f32(p + "q.b"), f32(p + "k.b"), f32(p + "v.b")]),
      q_norm=f32(p + "q.norm"), k_norm=f32(p + "k.norm"),
      dist_bias=rel[buckets].contiguous(),  # [window, H]
      head_bias=f32(p + "pb"), talk=f32(p + "talk").contiguous(),
      wo=t[p + "o"], w_gate_up=None, w_down=None,
  )
  for name, shape in (("wqkv", (H * d + G * d + G * dv, config.emb_dim)), ("wo", (config.emb_dim, H * dv)), ("talk", (H, H)),
                      ("q_norm", (d,)), ("k_norm", (d,)), ("head_bias", (H,))):
    if tuple(plan[name].shape) != shape:
      raise ValueError(f"layer {i}: {name} has shape {tuple(plan[name].shape)}, expected {shape}")
  if m.get("v_mix"):
    plan["value_mix"] = 1 if i == first_mix else 2
    plan["value_lambda"] = 0.0 if i == first_mix else float(f32(p + "vmix"))
  if spec.get("mlp"):
    F = int(spec["mlp"]["ff"])
    gate, up = t[f"l{i}.mlp.gate"], t[f"l{i}.mlp.up"]
    if tuple(gate.shape) != (F, config.emb_dim) or tuple(up.shape) != (F, config.emb_dim):
      raise ValueError(f"layer {i}: feed-forward matrices do not match ff = {F}")
    plan.update(ff=F, gain2=float(f32(f"l{i}.norm2")), w_down=t[f"l{i}.mlp.down"],
                w_gate_up=torch.stack([gate, up], dim=1).reshape(2 * F, config.emb_dim))  # row 2f = gate f, row 2f + 1 = up f
  return plan


def model_plan(config, tensors: Dict[str, torch.Tensor]) -> Dict[str, Any]:
  specs = config.layer_specs
  mixing = [i for i, l in enumerate(specs) if l["mixer"].get("v_mix")]
  first_mix = mixing[0] if mixing else -1
  return dict(
      embedding=tensors["embed"], head=tensors["head"], final_gain=float(tensors["final.norm"].to(torch.float32)),
      embed_scale=float(config.embedding_scale),
      layers=[layer_plan(config, tensors, i, first_mix) for i in range(len(specs))],
  )


def random_tensors(config, seed: int = 0, device: Any = "cpu", bias_rows: int = 32) -> Dict[str, torch.Tensor]:
  """Random bf16 weights with the design's tensor names, for `config` (benchmarks and smoke runs; made on `device`)."""
  g = torch.Generator(device=device).manual_seed(seed)
  E, V = int(config.emb_dim), int(config.vocab_size)
  bf = torch.bfloat16

  def rn(*shape, std=1.0, mean=0.0):
    return (torch.randn(tuple(shape), generator=g, device=device) * std + mean).to(bf)

  t = {"embed": rn(V, E, std=1.0 / math.sqrt(E)), "final.norm": rn(std=0.05, mean=1.0), "head": rn(V, E, std=1.0 / math.sqrt(E))}
  for i, l in enumerate(config.layer_specs):
    m, p = l["mixer"], f"l{i}."
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    t[p + "norm1"] = rn(std=0.05, mean=0.5)
    for name, n in (("q", H * d), ("k", G * d), ("v", G * dv)):
      t[p + "mix." + name] = rn(n, E, std=1.0 / math.sqrt(E))
      t[p + "mix." + name + ".b"] = rn(n, std=0.1)
    t[p + "mix.q.norm"], t[p + "mix.k.norm"] = rn(d, std=0.1, mean=1.0), rn(d, std=0.1, mean=1.0)
    t[p + "mix.rel"] = rn(bias_rows, H, std=0.5)
    t[p + "mix.vmix"] = rn(std=0.05, mean=0.3)
    t[p + "mix.talk"] = (torch.eye(H, device=device) + 0.2 * torch.randn(H, H, generator=g, device=device)).to(bf)
    t[p + "mix.pb"] = rn(H, std=0.5, mean=-3.0)
    t[p + "mix.o"] = rn(E, H * dv, std=1.0 / math.sqrt(H * dv))
    if l.get("mlp"):
      F = int(l["mlp"]["ff"])
      t[p + "norm2"] = rn(std=0.05, mean=0.5)
      t[p + "mlp.gate"], t[p + "mlp.up"] = rn(F, E, std=1.0 / math.sqrt(E)), rn(F, E, std=1.0 / math.sqrt(E))
      t[p + "mlp.down"] = rn(E, F, std=1.0 / math.sqrt(F))
  return t


def model_dict(width: int, vocab: int, layers: List[dict], eps: float = 1e-5, embed_scale: float = 1.0) -> dict:
  """A config.json-shaped dict (tests, benchmarks)."""
  return {"architecture": "Kifusun", "width": width, "vocab": vocab, "norm": {"eps": eps}, "embedding": {"scale": embed_scale}, "layers": layers}


def attention_layer(heads: int, kv_heads: int, dim: int, vdim: int, window: int, ff: int = 0, v_mix: bool = True, softcap: float = 50.0,
                    bias_max: float = 128.0, scale: float = 0.0) -> dict:
  return {"type": "attention",
          "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window}, "scale": scale or dim**-0.5,
                    "softcap": softcap, "bias_max": bias_max, "v_mix": v_mix},
          "mlp": {"kind": "dense", "ff": ff} if ff else None}
