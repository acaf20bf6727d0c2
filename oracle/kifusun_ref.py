"""Plain, slow restatement of the Kifusun decoder (test infrastructure only; shares no code with the product path).

One function per mechanism, written from the design's equations in float64 unless a dtype is passed.  Notation:
``x`` the residual stream [T, E]; a layer does ``x += g1 * unit(mixer(x))`` then ``x += g2 * unit(ff(x))`` where
``unit(y) = y / sqrt(mean(y^2) + eps)`` and g1, g2 are single numbers; both sublayers read x itself.

The mixer is a sliding-window attention without softmax and without rotation:

  q, k, v      = Wq x + bq, Wk x + bk, Wv x + bv
  q, k         = per-head RMS norm with a weight vector shared by the heads
  s_g(i, j)    = cap * tanh(scale * <q_g(i), k_kv(g)(j)> / cap) + rel[bucket(i - j), g]        for 0 <= i - j < window
  w_g(i, j)    = sigmoid(s_g(i, j) + pb[g])
  w'_h(i, j)   = sum_g talk[h, g] w_g(i, j)
  out_h(i)     = sum_j w'_h(i, j) v_kv(h)(j)
  y            = Wo concat_h out_h

with ``v = (1 - lam) v + lam v_first`` in every value-mixing layer but the first one of the model (v_first = that first
layer's values of the same token).
"""

from __future__ import annotations

import math

import numpy as np
import torch


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
  return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z**3)))


def unit_rms(y: torch.Tensor, eps: float) -> torch.Tensor:
  return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps)


def scalar_norm(y: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
  return unit_rms(y, eps) * gain


def distance_bucket(n: int, rows: int, far: float) -> int:
  """Row of the distance-bias table for the distance n >= 0: exact below rows // 2, logarithmic up to `far`, then the last row."""
  half = rows // 2
  if n < half:
    return n
  return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def window_weights(q, k, rel, pb, talk, scale, cap, window, far, q_pos, k_pos):
  """q [Tq, H, d], k [Tk, G, d] (already normalised) -> mixed weights [H, Tq, Tk]; zero outside the window."""
  H, G = q.shape[1], k.shape[1]
  rep = H // G
  s = torch.einsum("ihd,jhd->hij", q, k.repeat_interleave(rep, dim=1)) * scale
  if cap:
    s = cap * torch.tanh(s / cap)
  dist = q_pos[:, None] - k_pos[None, :]
  seen = (dist >= 0) & (dist < window)
  rows = rel.shape[0]
  b = torch.tensor([[distance_bucket(int(d), rows, far) if d >= 0 else 0 for d in row] for row in dist.tolist()], dtype=torch.long)
  s = s + rel[b].permute(2, 0, 1)
  w = torch.sigmoid(s + pb[:, None, None]) * seen[None].to(s.dtype)
  return torch.einsum("hg,gij->hij", talk, w)


def head_norm(t: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
  return unit_rms(t, eps) * weight


class KifusunRef:
  """Whole-sequence forward and a token-by-token forward over a plain python cache."""

  def __init__(self, config: dict, tensors: dict, dtype=torch.float64):
    self.c = config
    self.t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    self.dtype = dtype
    self.eps = float(config["norm"]["eps"])
    mixing = [i for i, l in enumerate(config["layers"]) if l["mixer"].get("v_mix")]
    self.first_mix = mixing[0] if mixing else -1

  # -- pieces -----------------------------------------------------------------------------------
  def embed(self, tokens):
    return self.t["embed"][torch.as_tensor(tokens, dtype=torch.long)] * float(self.c["embedding"]["scale"])

  def qkv(self, i, x, v_first):
    m, p = self.c["layers"][i]["mixer"], f"l{i}.mix."
    t = self.t
    T = x.shape[0]
    q = (x @ t[p + "q"].T + t[p + "q.b"]).reshape(T, m["heads"], m["dim"])
    k = (x @ t[p + "k"].T + t[p + "k.b"]).reshape(T, m["kv_heads"], m["dim"])
    v = (x @ t[p + "v"].T + t[p + "v.b"]).reshape(T, m["kv_heads"], m["vdim"])
    q = head_norm(q, t[p + "q.norm"], self.eps)
    k = head_norm(k, t[p + "k.norm"], self.eps)
    if m.get("v_mix"):
      if i == self.first_mix:
        v_first = v
      else:
        lam = t[p + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    return q, k, v, v_first

  def attend(self, i, q, k, v, q_pos, k_pos):
    m, p = self.c["layers"][i]["mixer"], f"l{i}.mix."
    t = self.t
    w = window_weights(q, k, t[p + "rel"], t[p + "pb"], t[p + "talk"], float(m["scale"]), float(m.get("softcap") or 0.0),
                       int(m["mask"]["size"]), float(m["bias_max"]), q_pos, k_pos)
    rep = m["heads"] // m["kv_heads"]
    out = torch.einsum("hij,jhd->ihd", w, v.repeat_interleave(rep, dim=1))
    return out.reshape(q.shape[0], -1) @ t[p + "o"].T

  def ff(self, i, x):
    p = f"l{i}.mlp."
    t = self.t
    return (gelu_tanh(x @ t[p + "gate"].T) * (x @ t[p + "up"].T)) @ t[p + "down"].T

  def head(self, x):
    return scalar_norm(x, self.t["final.norm"], self.eps) @ self.t["head"].T

  # -- whole sequence ---------------------------------------------------------------------------
  def forward(self, tokens, return_layers=False):
    x = self.embed(tokens)
    pos = torch.arange(x.shape[0])
    v_first, layers = None, []
    for i, l in enumerate(self.c["layers"]):
      q, k, v, v_first = self.qkv(i, x, v_first)
      x = x + scalar_norm(self.attend(i, q, k, v, pos, pos), self.t[f"l{i}.norm1"], self.eps)
      if l.get("mlp"):
        x = x + scalar_norm(self.ff(i, x), self.t[f"l{i}.norm2"], self.eps)
      layers.append(x)
    logits = self.head(x)
    return (logits, torch.stack(layers)) if return_layers else logits

  # -- incremental: feed `tokens` after `cache` (a list of per-layer (k, v) with all earlier positions) ------
  def new_cache(self):
    return [None] * len(self.c["layers"])

  def extend(self, cache, tokens):
    start = 0 if cache[0] is None else cache[0][0].shape[0]
    x = self.embed(tokens)
    pos = torch.arange(start, start + x.shape[0])
    v_first = None
    for i, l in enumerate(self.c["layers"]):
      q, k, v, v_first = self.qkv(i, x, v_first)
      if cache[i] is not None:
        k, v = torch.cat([cache[i][0], k]), torch.cat([cache[i][1], v])
      cache[i] = (k, v)
      x = x + scalar_norm(self.attend(i, q, k, v, pos, torch.arange(k.shape[0])), self.t[f"l{i}.norm1"], self.eps)
      if l.get("mlp"):
        x = x + scalar_norm(self.ff(i, x), self.t[f"l{i}.norm2"], self.eps)
    return self.head(x)


def random_model(config: dict, seed: int = 0, bias_rows: int = 10) -> dict:
  """Random bf16 weights with the design's tensor names for `config` (a dict with the keys of its config.json)."""
  g = torch.Generator().manual_seed(seed)
  E, V = int(config["width"]), int(config["vocab"])
  bf = torch.bfloat16
  rn = lambda *shape, std=1.0: (torch.randn(*shape, generator=g) * std).to(bf)
  t = {"embed": rn(V, E, std=1.0 / math.sqrt(E)), "final.norm": (1.0 + 0.2 * torch.randn((), generator=g)).to(bf), "head": rn(V, E, std=1.0 / math.sqrt(E))}
  for i, l in enumerate(config["layers"]):
    m, p = l["mixer"], f"l{i}."
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rows = bias_rows
    t[p + "norm1"] = (0.7 + 0.2 * torch.randn((), generator=g)).to(bf)
    t[p + "mix.q"], t[p + "mix.q.b"] = rn(H * d, E, std=1.0 / math.sqrt(E)), rn(H * d, std=0.1)
    t[p + "mix.k"], t[p + "mix.k.b"] = rn(G * d, E, std=1.0 / math.sqrt(E)), rn(G * d, std=0.1)
    t[p + "mix.v"], t[p + "mix.v.b"] = rn(G * dv, E, std=1.0 / math.sqrt(E)), rn(G * dv, std=0.1)
    t[p + "mix.q.norm"] = (1.0 + 0.2 * torch.randn(d, generator=g)).to(bf)
    t[p + "mix.k.norm"] = (1.0 + 0.2 * torch.randn(d, generator=g)).to(bf)
    t[p + "mix.rel"] = rn(rows, H, std=0.5)
    t[p + "mix.vmix"] = torch.tensor(0.3 + 0.1 * i).to(bf)
    t[p + "mix.talk"] = (torch.eye(H) + 0.3 * torch.randn(H, H, generator=g)).to(bf)
    t[p + "mix.pb"] = (rn(H, std=0.5).float() - 2.0).to(bf)
    t[p + "mix.o"] = rn(E, H * dv, std=1.0 / math.sqrt(H * dv))
    if l.get("mlp"):
      F = l["mlp"]["ff"]
      t[p + "norm2"] = (0.7 + 0.2 * torch.randn((), generator=g)).to(bf)
      t[p + "mlp.gate"], t[p + "mlp.up"] = rn(F, E, std=1.0 / math.sqrt(E)), rn(F, E, std=1.0 / math.sqrt(E))
      t[p + "mlp.down"] = rn(E, F, std=1.0 / math.sqrt(F))
  return t


def small_config(layers=3, width=48, vocab=61, heads=4, kv_heads=2, dim=24, vdim=16, window=7, ff=40, bias_max=40,
                 softcap=30.0, v_mix=(True, True, True), mlp=(True, False, True), eps=1e-5, embed_scale=3.0):
  """A config dict in the layout of the design's config.json, with small sizes."""
  ls = []
  for i in range(layers):
    ls.append({"type": "attention",
               "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window}, "scale": dim**-0.5,
                         "softcap": softcap, "bias_max": bias_max, "v_mix": bool(v_mix[i % len(v_mix)])},
               "mlp": {"kind": "dense", "ff": ff} if mlp[i % len(mlp)] else None})
  return {"architecture": "Kifusun", "vocab": vocab, "width": width, "embedding": {"scale": embed_scale}, "norm": {"eps": eps}, "layers": ls}
