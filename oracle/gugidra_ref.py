"""Plain, slow restatement of the Gugidra decoder in numpy float64 (test infrastructure only; shares no code with the product
path).  One function per mechanism; every recurrence is written as the token-by-token loop it is defined by.

Notation.  ``x`` [T, E] is the residual stream, ``rms(y) = y / sqrt(mean(y^2) + eps)`` and ``wnorm(y, w) = rms(y) * (1 + w)``.
A layer is ``x += wnorm(mixer(wnorm(x, n1)), n1b)`` then, when it has a feed-forward, ``x += wnorm(ff(wnorm(x, n2)), n2b)``.
The layer list may hold a loop: layers [start, stop) run `times` times with the same weights and a state of their own per pass;
before pass t > 0 the scaled embedding is added again, and before every pass the vector ``loop.step[t]``.

Mixers (h [T, E] is the normed input):

* ``gla``: per head ``S_t = diag(a_t) S_{t-1} + k_t v_t^T``, ``o_t = S_t^T q_t`` with ``a = sigmoid(z)^(1/tau)``,
  ``z = A2 (A1 h) + b``; ``o`` is RMS-normed per head with a weight over vdim, gated by ``silu(G h)`` and projected.
* ``parallel``: ``ls * softmax_attention(h) + rs * mlstm(h)``.  The attention has grouped key heads, rotary positions on the
  first `rot.dims` channels of each head in the interleaved pairing, biases on q, k and the output, and its values are the
  keys before rotation.  The mLSTM keeps (S, n, m) per head with capped log gates and a running maximum that starts at 0.

Feed-forwards: ``down(act(gate h, up h))`` with ``act(g, u) = g' sigmoid(1.702 g') (u' + 1)``, ``g' = min(g, L)``,
``u' = clip(u, -L, L)``; or a mixture of such experts with a sigmoid router, a correction that only steers the choice, a
restriction to the best groups, weights renormalised over the chosen experts, and a shared expert that every token uses.
"""

from __future__ import annotations

import math

import numpy as np

F = np.float64


def rms(y: np.ndarray, eps: float) -> np.ndarray:
  return y / np.sqrt((y * y).mean(axis=-1, keepdims=True) + eps)


def wnorm(y: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
  return rms(y, eps) * (1.0 + w)


def sigmoid(z):
  return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
  return -np.logaddexp(0.0, -z)


def clamped_gate(g: np.ndarray, u: np.ndarray, limit: float) -> np.ndarray:
  g = np.minimum(g, limit)
  u = np.clip(u, -limit, limit)
  return g * sigmoid(1.702 * g) * (u + 1.0)


def gated_ff(h, gate, up, down, limit):
  return clamped_gate(h @ gate.T, h @ up.T, limit) @ down.T


def rotate_pairs(t: np.ndarray, pos: np.ndarray, dims: int, base: float) -> np.ndarray:
  """t [T, heads, d]: channels (2i, 2i + 1), i < dims / 2, turn by pos * base^(-2i / dims); the rest stay."""
  out = t.copy()
  i = np.arange(dims // 2, dtype=F)
  ang = pos.astype(F)[:, None] * base ** (-2.0 * i / dims)[None, :]
  c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
  a, b = t[..., 0:dims:2], t[..., 1:dims:2]
  out[..., 0:dims:2] = a * c - b * s
  out[..., 1:dims:2] = b * c + a * s
  return out


def softmax_attention(q, k, v, q_pos, k_pos, scale):
  """q [Tq, H, d], k [Tk, G, d], v [Tk, G, dv] -> [Tq, H, dv]; a query sees the keys at positions <= its own."""
  H, G = q.shape[1], k.shape[1]
  out = np.zeros((q.shape[0], H, v.shape[2]), F)
  seen = k_pos[None, :] <= q_pos[:, None]
  for h in range(H):
    g = h // (H // G)
    s = (q[:, h] @ k[:, g].T) * scale
    s = np.where(seen, s, -np.inf)
    p = np.exp(s - s.max(axis=1, keepdims=True))
    out[:, h] = (p / p.sum(axis=1, keepdims=True)) @ v[:, g]
  return out


def gla_scan(q, k, v, a, S):
  """q, k, a [T, H, d], v [T, H, dv], S [H, d, dv] (updated in place) -> o [T, H, dv]."""
  o = np.zeros(v.shape, F)
  for t in range(q.shape[0]):
    for h in range(q.shape[1]):
      S[h] = a[t, h][:, None] * S[h] + np.outer(k[t, h], v[t, h])
      o[t, h] = S[h].T @ q[t, h]
  return o


def mlstm_scan(q, k, v, ig, fg, S, n, m):
  """q, k [T, H, d], v [T, H, dv], log gates ig, fg [T, H]; state S [H, d, dv], n [H, d], m [H] (updated in place)."""
  o = np.zeros(v.shape, F)
  for t in range(q.shape[0]):
    for h in range(q.shape[1]):
      m_new = max(fg[t, h] + m[h], ig[t, h])
      keep, put = math.exp(fg[t, h] + m[h] - m_new), math.exp(ig[t, h] - m_new)
      S[h] = keep * S[h] + put * np.outer(k[t, h], v[t, h])
      n[h] = keep * n[h] + put * k[t, h]
      m[h] = m_new
      o[t, h] = (S[h].T @ q[t, h]) / (max(abs(float(n[h] @ q[t, h])), math.exp(-m_new)) + 1e-6)
  return o


def route(h, router, correction, top, groups, keep):
  """-> (chosen [T, top] expert indices, weights [T, top])."""
  s = sigmoid(h @ router.T)
  choice = s + correction[None, :]
  T, E = s.shape
  per = E // groups
  if groups > 1:
    gs = np.sort(choice.reshape(T, groups, per), axis=2)[:, :, -2:].sum(axis=2) if per >= 2 else choice.reshape(T, groups, per).sum(axis=2)
    best = np.argsort(-gs, axis=1, kind="stable")[:, :keep]
    ok = np.zeros((T, groups), bool)
    np.put_along_axis(ok, best, True, axis=1)
    choice = np.where(np.repeat(ok, per, axis=1), choice, -np.inf)
  chosen = np.argsort(-choice, axis=1, kind="stable")[:, :top]
  w = np.take_along_axis(s, chosen, axis=1)
  return chosen, w / (w.sum(axis=1, keepdims=True) + 1e-20)


class GugidraRef:
  """forward(tokens, state) runs the tokens of ONE sequence from `state` (new_state() at its start) and returns the logits
  [T, vocab]; feeding a sequence in pieces, or token by token, continues it."""

  def __init__(self, config: dict, tensors: dict):
    self.c = config
    self.t = {k: np.asarray(v, dtype=F) for k, v in tensors.items()}
    self.eps = float(config["norm"]["eps"])
    L = len(config["layers"])
    loop = config.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, n = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    self.runs = []  # (layer, pass number or -1, first layer of a pass)
    for i in range(a):
      self.runs.append((i, -1, False))
    for p in range(n if b > a else 0):
      for i in range(a, b):
        self.runs.append((i, p, i == a))
    for i in range(b if b > a else a, L):
      self.runs.append((i, -1, False))

  def new_state(self):
    st = []
    for i, _, _ in self.runs:
      l = self.c["layers"][i]
      m = l["mixer"]
      if l["type"] == "gla":
        st.append({"S": np.zeros((m["heads"], m["dim"], m["vdim"]), F)})
      else:
        r, a = m["right"], m["left"]
        st.append({"S": np.zeros((r["heads"], r["dim"], r["vdim"]), F), "n": np.zeros((r["heads"], r["dim"]), F), "m": np.zeros(r["heads"], F),
                   "k": np.zeros((0, a["kv_heads"], a["dim"]), F), "v": np.zeros((0, a["kv_heads"], a["dim"]), F)})
    return {"pos": 0, "layers": st}

  # -- mixers -----------------------------------------------------------------------------------
  def gla(self, i, h, st):
    m, t, p = self.c["layers"][i]["mixer"], self.t, f"l{i}.mix."
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ t[p + "q"].T * d**-0.5).reshape(T, H, d)
    k = (h @ t[p + "k"].T).reshape(T, H, d)
    v = (h @ t[p + "v"].T).reshape(T, H, dv)
    z = (h @ t[p + "a1"].T) @ t[p + "a2"].T + t[p + "a2.b"]
    a = np.exp(log_sigmoid(z) / float(m["tau"])).reshape(T, H, d)
    o = gla_scan(q, k, v, a, st["S"])
    o = rms(o, self.eps) * t[p + "norm"][None, None, :]
    g = h @ t[p + "g"].T
    return (o.reshape(T, H * dv) * (g * sigmoid(g))) @ t[p + "o"].T

  def attention(self, i, h, pos, st):
    m, t, p = self.c["layers"][i]["mixer"]["left"], self.t, f"l{i}.mix.left."
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    T = h.shape[0]
    q = (h @ t[p + "q"].T + t[p + "q.b"]).reshape(T, H, d)
    k = (h @ t[p + "k"].T + t[p + "k.b"]).reshape(T, G, d)
    st["v"] = np.concatenate([st["v"], k], axis=0)
    rd, rb = int(m["rot"]["dims"]), float(m["rot"]["base"])
    st["k"] = np.concatenate([st["k"], rotate_pairs(k, pos, rd, rb)], axis=0)
    o = softmax_attention(rotate_pairs(q, pos, rd, rb), st["k"], st["v"], pos, np.arange(st["k"].shape[0]), float(m["scale"]))
    return o.reshape(T, H * d) @ t[p + "o"].T + t[p + "o.b"]

  def mlstm(self, i, h, st):
    m, t, p = self.c["layers"][i]["mixer"]["right"], self.t, f"l{i}.mix.right."
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    T = h.shape[0]
    q = (h @ t[p + "q"].T * d**-0.5).reshape(T, H, d)
    k = (h @ t[p + "k"].T).reshape(T, H, d)
    v = (h @ t[p + "v"].T).reshape(T, H, dv)
    ig = cap * np.tanh((h @ t[p + "i"].T + t[p + "i.b"]) / cap)
    fg = log_sigmoid(cap * np.tanh((h @ t[p + "f"].T + t[p + "f.b"]) / cap))
    o = rms(mlstm_scan(q, k, v, ig, fg, st["S"], st["n"], st["m"]), self.eps)
    return (o.reshape(T, H * dv) * t[p + "norm"][None, :] * sigmoid(h @ t[p + "g"].T)) @ t[p + "o"].T

  def mixer(self, i, h, pos, st):
    l = self.c["layers"][i]
    if l["type"] == "gla":
      return self.gla(i, h, st)
    if l["type"] == "parallel":
      m = l["mixer"]
      return float(m["left_scale"]) * self.attention(i, h, pos, st) + float(m["right_scale"]) * self.mlstm(i, h, st)
    raise ValueError(l["type"])

  # -- feed-forwards ----------------------------------------------------------------------------
  def ff(self, i, h):
    f, t, p = self.c["layers"][i]["mlp"], self.t, f"l{i}.mlp."
    if f["kind"] == "dense":
      return gated_ff(h, t[p + "gate"], t[p + "up"], t[p + "down"], float(f["limit"]))
    r = f["router"]
    chosen, w = route(h, t[p + "router"], t[p + "correction"], int(r["top"]), int(r["groups"]["count"]), int(r["groups"]["keep"]))
    y = np.zeros(h.shape, F)
    for row in range(h.shape[0]):
      for e, we in zip(chosen[row], w[row]):
        q = f"{p}e{int(e)}."
        y[row] += we * gated_ff(h[row : row + 1], t[q + "gate"], t[q + "up"], t[q + "down"], float(f["expert"]["limit"]))[0]
    if f.get("shared"):
      y += gated_ff(h, t[p + "shared.gate"], t[p + "shared.up"], t[p + "shared.down"], float(f["shared"]["limit"]))
    return y

  # -- the model --------------------------------------------------------------------------------
  def forward(self, tokens, state, layer_outputs=None):
    t, eps = self.t, self.eps
    T = len(tokens)
    pos = np.arange(state["pos"], state["pos"] + T)
    x0 = t["embed"][np.asarray(tokens)] * float(self.c["embedding"]["scale"])
    x = x0.copy()
    for r, (i, p, first) in enumerate(self.runs):
      if first:
        if p > 0:
          x = x + x0
        x = x + t["loop.step"][p][None, :]
      l, n = self.c["layers"][i], f"l{i}."
      x = x + wnorm(self.mixer(i, wnorm(x, t[n + "norm1"], eps), pos, state["layers"][r]), t[n + "norm1b"], eps)
      if l.get("mlp"):
        x = x + wnorm(self.ff(i, wnorm(x, t[n + "norm2"], eps)), t[n + "norm2b"], eps)
      if layer_outputs is not None:
        layer_outputs.append(x.copy())
    state["pos"] += T
    cap = float(self.c["logit_softcap"])
    z = wnorm(x, t["final.norm"], eps) @ t["head"].T
    return cap * np.tanh(z / cap) if cap else z


def logits_of(config: dict, tensors: dict, tokens) -> np.ndarray:
  """The logits [T, vocab] of one sequence fed at once."""
  ref = GugidraRef(config, tensors)
  return ref.forward(list(tokens), ref.new_state())


def on_bf16_grid(a) -> np.ndarray:
  """`a` rounded (to nearest, ties to even) to numbers that bfloat16 represents exactly, as float64."""
  u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
  u = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
  return u.view(np.float32).astype(F)


def random_model(config: dict, seed: int = 0, rank: int = 5) -> dict:
  """Random weights with the design's tensor names as float64 arrays that are exactly representable in bfloat16, so that an
  engine loading them as bfloat16 computes with the same numbers."""
  rng = np.random.Generator(np.random.PCG64(seed))
  E, V = int(config["width"]), int(config["vocab"])
  rn = lambda *shape, std=1.0, mean=0.0: rng.standard_normal(shape) * std + mean
  lin = lambda n, k: rn(n, k, std=k**-0.5)
  t = {"embed": rn(V, E), "final.norm": rn(E, std=0.2), "head": lin(V, E)}
  if config.get("loop"):
    t["loop.step"] = rn(int(config["loop"]["times"]), E, std=0.5)
  for i, l in enumerate(config["layers"]):
    p, m = f"l{i}.", l["mixer"]
    for n in ("norm1", "norm1b", "norm2", "norm2b"):
      t[p + n] = rn(E, std=0.2)
    if l["type"] == "gla":
      H, d, dv = m["heads"], m["dim"], m["vdim"]
      q = p + "mix."
      t[q + "q"], t[q + "k"], t[q + "v"], t[q + "g"] = lin(H * d, E), lin(H * d, E), lin(H * dv, E), lin(H * dv, E)
      t[q + "o"], t[q + "norm"] = lin(E, H * dv), rn(dv, std=0.2, mean=1.0)
      t[q + "a1"], t[q + "a2"], t[q + "a2.b"] = lin(rank, E), rn(H * d, rank, std=1.0), rn(H * d, std=1.5, mean=1.0)
    else:
      a, r = m["left"], m["right"]
      H, G, d = a["heads"], a["kv_heads"], a["dim"]
      q = p + "mix.left."
      t[q + "q"], t[q + "k"], t[q + "o"] = lin(H * d, E), lin(G * d, E), lin(E, H * d)
      t[q + "q.b"], t[q + "k.b"], t[q + "o.b"] = rn(H * d, std=0.3), rn(G * d, std=0.3), rn(E, std=0.3)
      Hr, dr, dvr = r["heads"], r["dim"], r["vdim"]
      q = p + "mix.right."
      t[q + "q"], t[q + "k"], t[q + "v"], t[q + "g"] = lin(Hr * dr, E), lin(Hr * dr, E), lin(Hr * dvr, E), lin(Hr * dvr, E)
      t[q + "o"], t[q + "norm"] = lin(E, Hr * dvr), rn(Hr * dvr, std=0.2, mean=1.0)
      t[q + "i"], t[q + "f"] = lin(Hr, E) * 2.0, lin(Hr, E) * 2.0
      t[q + "i.b"], t[q + "f.b"] = rn(Hr, std=1.0), rn(Hr, std=1.0, mean=2.0)
    f = l.get("mlp")
    if not f:
      continue
    q = p + "mlp."

    def gated(prefix, n):
      t[prefix + "gate"], t[prefix + "up"], t[prefix + "down"] = lin(n, E) * 2.0, lin(n, E) * 2.0, lin(E, n)

    if f["kind"] == "dense":
      gated(q, f["ff"])
    else:
      n_exp = f["router"]["experts"]
      for e in range(n_exp):
        gated(f"{q}e{e}.", f["expert"]["ff"])
      t[q + "router"], t[q + "correction"] = lin(n_exp, E) * 3.0, rn(n_exp, std=0.3)
      if f.get("shared"):
        gated(q + "shared.", f["shared"]["ff"])
  return {k: on_bf16_grid(v) for k, v in t.items()}
