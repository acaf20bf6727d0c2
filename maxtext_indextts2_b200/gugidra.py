"""The Gugidra design: a decoder whose config.json lists its layers one by one, with recurrent and attention mixers, routed
feed-forwards and a loop over a span of layers.

A layer is ``x += wnorm(mixer(wnorm(x, n1)), n1b)`` then (if it has one) ``x += wnorm(ff(wnorm(x, n2)), n2b)`` with
``wnorm(y, w) = y / sqrt(mean(y^2) + eps) * (1 + w)``.  Mixers:

* ``gla``      -- gated linear attention: a matrix state per head that decays per key channel (a low-rank projection, a sigmoid
                  taken to the power 1 / tau), a per-head RMS norm of the read-out, a silu gate;
* ``parallel`` -- the weighted sum of a causal softmax attention (grouped key heads, rotary positions on interleaved channel
                  pairs, biased projections, values = the un-rotated keys) and an mLSTM (matrix memory with capped log gates and
                  a running maximum), both reading the same normed input.

Feed-forwards: a clamped gated form ``down(g sigmoid(1.702 g) (u + 1))``, dense or as a mixture of experts (sigmoid router, a
correction that only steers the choice, groups of experts of which the best are kept, a shared expert).  ``loop`` repeats the
layers [start, stop) `times` times with the same weights; every pass has its own cache and state, and before a pass the scaled
embedding (from the second pass on) and a learned vector per pass are added to the stream.  The logits are soft-capped.

This module is the design's entry in the framework: config.json -> config keys (`config_keys`), checks (`validate_layer_specs`),
safetensors names -> the layer-run descriptors of the layered engine (`model_plan`; a looped layer is listed once per pass), and
random weights of any size (`random_tensors`).  No arithmetic of the model happens here: on the device a ``gla`` layer is a
composite mixer with a recurrence only, a ``parallel`` layer one with an attention and a recurrence.
"""

from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Tuple

import numpy as np
import torch

MIXERS = ("gla", "parallel")
FF_KINDS = ("dense", "moe")
MLSTM_DENOM_EPS = 1e-6   # added to the mLSTM's denominator
GATE_SLOPE = 1.702       # (fixed in the kernels' clamped gate: g * sigmoid(1.702 g) * (u + 1))
TILE_ROWS = 128          # input-projection rows are padded with zero rows to whole tiles of the tensor-core GEMM


def layer_runs(n_layers: int, loop: Optional[dict]) -> List[Tuple[int, int, bool]]:
  """[(layer, pass number or -1, first of its pass)] in execution order."""
  if not loop or int(loop["stop"]) <= int(loop["start"]) or int(loop["times"]) < 1:
    return [(i, -1, False) for i in range(n_layers)]
  a, b, n = int(loop["start"]), int(loop["stop"]), int(loop["times"])
  runs = [(i, -1, False) for i in range(a)]
  for p in range(n):
    runs += [(i, p, i == a) for i in range(a, b)]
  return runs + [(i, -1, False) for i in range(b, n_layers)]


def config_keys(model: dict) -> dict:
  """config.json of a Gugidra model -> keys of configs/base.yml."""
  layers = model["layers"]
  validate_layer_specs(layers, model.get("loop"))
  ffs = []
  for l in layers:
    f = l.get("mlp")
    if f:
      ffs.append(int(f["ff"]) if f.get("kind", "dense") == "dense" else int(f["expert"]["ff"]))
  heads = [int(l["mixer"]["left"]["heads"]) if l["type"] == "parallel" else int(l["mixer"]["heads"]) for l in layers]
  return dict(
      base_emb_dim=int(model["width"]),
      vocab_size=int(model["vocab"]),
      base_num_decoder_layers=len(layers),
      global_parameter_scale=1,
      normalization_layer_epsilon=float(model["norm"]["eps"]),
      embedding_scale=float(model["embedding"]["scale"]),
      final_logits_soft_cap=float(model.get("logit_softcap") or 0.0),
      layer_specs=layers,
      layer_loop=dict(model["loop"]) if model.get("loop") else None,
      # (the homogeneous keys describe the first layer; the engine reads layer_specs)
      base_num_query_heads=heads[0],
      base_num_kv_heads=heads[0],
      head_dim=int(layers[0]["mixer"]["left"]["dim"]) if layers[0]["type"] == "parallel" else int(layers[0]["mixer"]["dim"]),
      base_mlp_dim=max(ffs) if ffs else 0,
  )


def _need(d: dict, keys, where: str) -> None:
  for k in keys:
    if k not in d:
      raise ValueError(f"{where}.{k} is missing")


def validate_layer_specs(specs: List[dict], loop: Optional[dict] = None) -> None:
  for i, l in enumerate(specs):
    if l.get("type") not in MIXERS:
      raise ValueError(f"layer {i}: mixer type {l.get('type')!r}; this design has {MIXERS}")
    m = l["mixer"]
    if l["type"] == "gla":
      _need(m, ("heads", "dim", "vdim", "tau"), f"layer {i}: mixer")
      if float(m["tau"]) <= 0:
        raise ValueError(f"layer {i}: tau must be positive")
    else:
      _need(m, ("left", "right", "left_scale", "right_scale"), f"layer {i}: mixer")
      a, r = m["left"], m["right"]
      _need(a, ("heads", "kv_heads", "dim", "vdim", "rot", "scale"), f"layer {i}: mixer.left")
      _need(r, ("heads", "dim", "vdim", "gate_cap"), f"layer {i}: mixer.right")
      if int(a["heads"]) % int(a["kv_heads"]):
        raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
      if int(a["vdim"]) != int(a["dim"]):
        raise ValueError(f"layer {i}: the attention's values are its keys, so vdim must equal dim")
      rd = int(a["rot"]["dims"])
      if rd % 2 or rd > int(a["dim"]):
        raise ValueError(f"layer {i}: rot.dims must be even and at most dim")
    f = l.get("mlp")
    if f is None:
      continue
    kind = f.get("kind", "dense")
    if kind not in FF_KINDS:
      raise ValueError(f"layer {i}: feed-forward kind {kind!r}; this design has {FF_KINDS}")
    if kind == "dense":
      _need(f, ("ff", "limit"), f"layer {i}: mlp")
    else:
      _need(f, ("expert", "router"), f"layer {i}: mlp")
      r = f["router"]
      E, top, gc, gk = int(r["experts"]), int(r["top"]), int(r["groups"]["count"]), int(r["groups"]["keep"])
      if E % gc or not 1 <= gk <= gc or not 1 <= top <= gk * (E // gc):
        raise ValueError(f"layer {i}: {E} experts, top {top}, {gc} groups of which {gk} are kept do not fit together")
  if loop:
    a, b, n = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    if not (0 <= a <= b <= len(specs)) or n < 1:
      raise ValueError(f"loop {loop} does not fit {len(specs)} layers")


def _interleave(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
  """[F, E], [F, E] -> [2F, E] with row 2f = gate f, row 2f + 1 = up f (the gated epilogue of the projections reads pairs)."""
  return torch.stack([gate, up], dim=1).reshape(2 * gate.shape[0], gate.shape[1])


def _shape(t: torch.Tensor, shape, name: str) -> torch.Tensor:
  if tuple(t.shape) != tuple(shape):
    raise ValueError(f"{name} has shape {tuple(t.shape)}, expected {tuple(shape)}")
  return t


def rot_frequencies(dims: int, base: float) -> torch.Tensor:
  """Radians per position of the channel pair i < dims / 2: base^(-2i / dims), in float64 (the device multiplies it by the
  position in double and reduces the angle before the fp32 sine and cosine)."""
  i = np.arange(dims // 2, dtype=np.float64)
  return torch.from_numpy(float(base) ** (-2.0 * i / dims))


def layer_plan(config, tensors: Dict[str, torch.Tensor], i: int) -> Dict[str, Any]:
  """What layer i hands to the layered engine: sizes and scalars (python numbers) and host tensors; matrices keep their stored
  dtype.  The input projections of the mixer are concatenated in the order the device reads them (attention q, k; recurrence q,
  k, v, output gate, then the decay's down-projection or the two gates' rows)."""
  spec = config.layer_specs[i]
  E = int(config.emb_dim)
  t, p = tensors, f"l{i}.mix."
  dev = tensors["embed"].device
  f32 = lambda name: t[name].to(torch.float32)
  rows: List[torch.Tensor] = []
  bias: List[torch.Tensor] = []
  has_bias = False

  def add(name: str, n: int, with_bias: bool = False):
    nonlocal has_bias
    rows.append(_shape(t[name], (n, E), name))
    if with_bias:
      bias.append(_shape(f32(name + ".b"), (n,), name + ".b"))
      has_bias = True
    else:
      bias.append(torch.zeros(n, dtype=torch.float32, device=dev))

  plan: Dict[str, Any] = dict(mixer="composite", norm_style="sandwich", attn=None, rec=None, ff_kind="none", ff=0, moe=None, bo=None)
  wo: List[torch.Tensor] = []
  m = spec["mixer"]
  if spec["type"] == "parallel":
    a, r = m["left"], m["right"]
    H, G, d, dv = int(a["heads"]), int(a["kv_heads"]), int(a["dim"]), int(a["vdim"])
    add(p + "left.q", H * d, True)
    add(p + "left.k", G * d, True)
    ls, rs = float(m["left_scale"]), float(m["right_scale"])
    plan["attn"] = dict(heads=H, kv_heads=G, dim=d, vdim=dv, window=0, rot_dims=int(a["rot"]["dims"]), values_are_keys=1,
                        scale=float(a["scale"]), out_scale=ls, rot_freq=rot_frequencies(int(a["rot"]["dims"]), float(a["rot"]["base"])))
    wo.append(_shape(t[p + "left.o"], (E, H * dv), p + "left.o"))
    plan["bo"] = _shape(f32(p + "left.o.b"), (E,), p + "left.o.b") * ls
    q = p + "right."
    Hr, dr, dvr = int(r["heads"]), int(r["dim"]), int(r["vdim"])
    for name, n in (("q", Hr * dr), ("k", Hr * dr), ("v", Hr * dvr), ("g", Hr * dvr)):
      add(q + name, n)
    rows.append(torch.cat([_shape(t[q + "i"], (Hr, E), q + "i"), _shape(t[q + "f"], (Hr, E), q + "f")], dim=0))
    bias.append(torch.zeros(2 * Hr, dtype=torch.float32, device=dev))  # (the gates' biases are added in fp32 by the recurrence)
    plan["rec"] = dict(kind="mlstm", heads=Hr, dim=dr, vdim=dvr, decay_rank=0, gate_silu=0, q_scale=dr**-0.5, tau=1.0,
                       gate_cap=float(r["gate_cap"]), denom_eps=MLSTM_DENOM_EPS, out_scale=rs,
                       gate_bias=torch.cat([_shape(f32(q + "i.b"), (Hr,), q + "i.b"), _shape(f32(q + "f.b"), (Hr,), q + "f.b")]),
                       out_norm=_shape(f32(q + "norm"), (Hr * dvr,), q + "norm"))
    wo.append(_shape(t[q + "o"], (E, Hr * dvr), q + "o"))
  else:
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    for name, n in (("q", H * d), ("k", H * d), ("v", H * dv), ("g", H * dv)):
      add(p + name, n)
    rank = int(t[p + "a1"].shape[0])
    add(p + "a1", rank)
    plan["rec"] = dict(kind="gla", heads=H, dim=d, vdim=dv, decay_rank=rank, gate_silu=1, q_scale=d**-0.5, tau=float(m["tau"]),
                       gate_cap=0.0, denom_eps=0.0, out_scale=1.0,
                       decay_up_t=_shape(f32(p + "a2"), (H * d, rank), p + "a2").t().contiguous(),
                       decay_bias=_shape(f32(p + "a2.b"), (H * d,), p + "a2.b"),
                       out_norm=_shape(f32(p + "norm"), (dv,), p + "norm").repeat(H))
    wo.append(_shape(t[p + "o"], (E, H * dv), p + "o"))
  w_in, b_in = torch.cat(rows, dim=0), torch.cat(bias)
  pad = (-w_in.shape[0]) % TILE_ROWS
  if pad and E % 64 == 0:
    w_in = torch.cat([w_in, torch.zeros(pad, E, dtype=w_in.dtype, device=dev)], dim=0)
    b_in = torch.cat([b_in, torch.zeros(pad, device=dev)])
  plan.update(w_in=w_in, b_in=b_in if has_bias else None, n_in=int(w_in.shape[0]), wo=torch.cat(wo, dim=1))
  for n in ("norm1", "norm1b"):
    plan[n] = _shape(f32(f"l{i}.{n}"), (E,), f"l{i}.{n}")
  f = spec.get("mlp")
  if f is not None:
    for n in ("norm2", "norm2b"):
      plan[n] = _shape(f32(f"l{i}.{n}"), (E,), f"l{i}.{n}")
    q = f"l{i}.mlp."

    def gated(prefix: str, F: int):
      return (_interleave(_shape(t[prefix + "gate"], (F, E), prefix + "gate"), _shape(t[prefix + "up"], (F, E), prefix + "up")),
              _shape(t[prefix + "down"], (E, F), prefix + "down"))

    if f.get("kind", "dense") == "dense":
      F = int(f["ff"])
      gu, dn = gated(q, F)
      plan.update(ff_kind="clamped", ff=F, ff_limit=float(f["limit"]), w_gate_up=gu, w_down=dn)
    else:
      r, ex, sh = f["router"], f["expert"], f.get("shared")
      n_exp, F = int(r["experts"]), int(ex["ff"])
      parts = [gated(f"{q}e{e}.", F) for e in range(n_exp)]
      moe = dict(experts=n_exp, top=int(r["top"]), groups=int(r["groups"]["count"]), keep_groups=int(r["groups"]["keep"]), ff=F,
                 limit=float(ex["limit"]), shared_ff=0, shared_limit=0.0,
                 w_router=_shape(t[q + "router"], (n_exp, E), q + "router"),
                 correction=_shape(f32(q + "correction"), (n_exp,), q + "correction") if (q + "correction") in t else None,
                 w_gate_up=torch.stack([g for g, _ in parts]), w_down=torch.stack([d_ for _, d_ in parts]),
                 shared_gate_up=None, shared_down=None)
      if sh:
        gu, dn = gated(q + "shared.", int(sh["ff"]))
        moe.update(shared_ff=int(sh["ff"]), shared_limit=float(sh["limit"]), shared_gate_up=gu, shared_down=dn)
      plan.update(ff_kind="moe", moe=moe)
  return plan


def model_plan(config, tensors: Dict[str, torch.Tensor]) -> Dict[str, Any]:
  """The engine's list of layer RUNS: a looped layer appears once per pass, sharing its weight tensors (``weights`` names the
  layer whose packed weights a run uses) and owning its pools and state."""
  specs = config.layer_specs
  E = int(config.emb_dim)
  loop = config.layer_loop
  runs = layer_runs(len(specs), loop)
  plans = {i: layer_plan(config, tensors, i) for i in sorted({i for i, _, _ in runs})}
  step = None
  if loop and any(p >= 0 for _, p, _ in runs):
    step = _shape(tensors["loop.step"].to(torch.float32), (int(loop["times"]), E), "loop.step")
  layers = []
  for i, p, first in runs:
    run = dict(plans[i])
    run["weights"] = i
    run["add_embedding"] = 1 if (first and p > 0) else 0
    run["add_vector"] = step[p].contiguous() if first else None
    layers.append(run)
  return dict(
      embedding=tensors["embed"], head=tensors["head"], final_gain=1.0, final_norm=_shape(tensors["final.norm"].to(torch.float32), (E,), "final.norm"),
      embed_scale=float(config.embedding_scale), logit_softcap=float(config.final_logits_soft_cap or 0.0), layers=layers,
  )


def random_tensors(config, seed: int = 0, device: Any = "cpu") -> Dict[str, torch.Tensor]:
  """Random bf16 weights with the design's tensor names, for `config` (tests, benchmarks and smoke runs; made on `device`)."""
  g = torch.Generator(device=device).manual_seed(seed)
  E, V = int(config.emb_dim), int(config.vocab_size)
  bf = torch.bfloat16

  def rn(*shape, std=1.0, mean=0.0):
    return (torch.randn(tuple(shape), generator=g, device=device) * std + mean).to(bf)

  lin = lambda n, k: rn(n, k, std=1.0 / math.sqrt(k))
  t = {"embed": rn(V, E), "final.norm": rn(E, std=0.1), "head": lin(V, E)}
  loop = config.layer_loop
  if loop:
    t["loop.step"] = rn(int(loop["times"]), E, std=0.3)
  for i, l in enumerate(config.layer_specs):
    p, m = f"l{i}.", l["mixer"]
    for n in ("norm1", "norm1b", "norm2", "norm2b"):
      t[p + n] = rn(E, std=0.1)
    if l["type"] == "gla":
      H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
      rank = int(m.get("rank", 16))
      q = p + "mix."
      t[q + "q"], t[q + "k"], t[q + "v"], t[q + "g"] = lin(H * d, E), lin(H * d, E), lin(H * dv, E), lin(H * dv, E)
      t[q + "o"], t[q + "norm"] = lin(E, H * dv), rn(dv, std=0.1, mean=1.0)
      t[q + "a1"], t[q + "a2"], t[q + "a2.b"] = lin(rank, E), rn(H * d, rank, std=0.5), rn(H * d, std=1.0, mean=2.0)
    else:
      a, r = m["left"], m["right"]
      H, G, d = int(a["heads"]), int(a["kv_heads"]), int(a["dim"])
      q = p + "mix.left."
      t[q + "q"], t[q + "k"], t[q + "o"] = lin(H * d, E), lin(G * d, E), lin(E, H * d)
      t[q + "q.b"], t[q + "k.b"], t[q + "o.b"] = rn(H * d, std=0.1), rn(G * d, std=0.1), rn(E, std=0.1)
      Hr, dr, dvr = int(r["heads"]), int(r["dim"]), int(r["vdim"])
      q = p + "mix.right."
      t[q + "q"], t[q + "k"], t[q + "v"], t[q + "g"] = lin(Hr * dr, E), lin(Hr * dr, E), lin(Hr * dvr, E), lin(Hr * dvr, E)
      t[q + "o"], t[q + "norm"] = lin(E, Hr * dvr), rn(Hr * dvr, std=0.1, mean=1.0)
      t[q + "i"], t[q + "f"] = lin(Hr, E), lin(Hr, E)
      t[q + "i.b"], t[q + "f.b"] = rn(Hr, std=0.5), rn(Hr, std=0.5, mean=3.0)
    f = l.get("mlp")
    if not f:
      continue
    q = p + "mlp."

    def gated(prefix, F):
      t[prefix + "gate"], t[prefix + "up"], t[prefix + "down"] = lin(F, E), lin(F, E), lin(E, F)

    if f.get("kind", "dense") == "dense":
      gated(q, int(f["ff"]))
    else:
      n_exp = int(f["router"]["experts"])
      for e in range(n_exp):
        gated(f"{q}e{e}.", int(f["expert"]["ff"]))
      t[q + "router"], t[q + "correction"] = lin(n_exp, E), rn(n_exp, std=0.2)
      if f.get("shared"):
        gated(q + "shared.", int(f["shared"]["ff"]))
  return t


# -- config.json-shaped dicts (tests, benchmarks) ----------------------------------------------------------------------------


def model_dict(width: int, vocab: int, layers: List[dict], eps: float = 1e-6, embed_scale: float = 1.0, logit_softcap: float = 30.0,
               loop: Optional[dict] = None) -> dict:
  out = {"architecture": "Gugidra", "width": width, "vocab": vocab, "norm": {"eps": eps}, "embedding": {"scale": embed_scale},
         "logit_softcap": logit_softcap, "layers": layers}
  if loop:
    out["loop"] = loop
  return out


def dense_ff(ff: int, limit: float = 7.0) -> dict:
  return {"kind": "dense", "ff": ff, "limit": limit}


def moe_ff(experts: int, top: int, ff: int, groups: int = 1, keep: int = 1, limit: float = 7.0, shared_ff: int = 0, shared_limit: float = 7.0) -> dict:
  out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}}
  if shared_ff:
    out["shared"] = {"ff": shared_ff, "limit": shared_limit}
  return out


def gla_layer(heads: int, dim: int, vdim: int, tau: float = 16.0, mlp: Optional[dict] = None, rank: int = 16) -> dict:
  return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}, "mlp": mlp}


def parallel_layer(heads: int, kv_heads: int, dim: int, r_heads: int, r_dim: int, r_vdim: int, mlp: Optional[dict] = None, rot_dims: Optional[int] = None,
                   rot_base: float = 10000.0, scale: float = 0.0, gate_cap: float = 15.0, left_scale: float = 1.0, right_scale: float = 1.0) -> dict:
  return {"type": "parallel",
          "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "rot": {"dims": dim if rot_dims is None else rot_dims, "base": rot_base},
                             "scale": scale or dim**-0.5},
                    "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "gate_cap": gate_cap},
                    "left_scale": left_scale, "right_scale": right_scale},
          "mlp": mlp}
