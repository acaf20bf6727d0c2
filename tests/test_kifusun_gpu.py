"""The Kifusun design on the layered engine against the plain restatement in oracle/kifusun_ref.py (float64, same bf16 weights).

Small configurations with random weights; where random weights would hide a fault (a window that is one key off, a bias bucket,
a far key) the weights are made so that it shows.  float32 engines are compared tightly, bfloat16 ones within bf16 rounding.
"""

import copy
import math

import numpy as np
import pytest
import torch

from maxtext_indextts2_b200 import maxengine, offline_engine, pyconfig
from oracle import kifusun_ref as ref

pytestmark = pytest.mark.gpu


def layer(heads=4, kv_heads=2, dim=24, vdim=16, window=7, ff=40, v_mix=True, softcap=30.0, bias_max=40.0, scale=None):
  return {"type": "attention",
          "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window},
                    "scale": scale if scale is not None else dim**-0.5, "softcap": softcap, "bias_max": bias_max, "v_mix": v_mix},
          "mlp": {"kind": "dense", "ff": ff} if ff else None}


def model(layers, width=48, vocab=61, eps=1e-5, embed_scale=3.0):
  return {"architecture": "Kifusun", "vocab": vocab, "width": width, "embedding": {"scale": embed_scale}, "norm": {"eps": eps}, "layers": layers}


def make_engine(cfg_dict, tensors, dtype="float32", slots=4, tokens_per_page=4, num_pages=40, max_len=128, **kw):
  config = pyconfig.from_model_dict(cfg_dict, dtype=dtype, per_device_batch_size=slots, max_target_length=max_len,
                                    pagedattn_tokens_per_page=tokens_per_page, pagedattn_num_pages=num_pages, **kw)
  engine = maxengine.MaxEngine(config)
  params = engine.load_params(tensors)
  engine.init_decode_state()
  return engine, params


def tokens_for(cfg_dict, n, seed=5):
  rng = np.random.Generator(np.random.PCG64(seed))
  return rng.integers(0, cfg_dict["vocab"], size=n).tolist()


def rel_err(got, want):
  return float((got - want).abs().max() / want.abs().max())


DEFAULT = lambda: model([layer(), layer(ff=0), layer(window=5)])


def whole(engine, toks, slot=0):
  out = engine.step([(slot, toks, list(range(len(toks))))]).cpu().double()
  engine.release_pages(slot)
  return out


# ---- each mechanism alone ------------------------------------------------------------------------------------------------------

def _neutral(t, cfg_dict):
  """Switch every optional mechanism of the mixer off in the weights: no distance bias, no head bias, identity head mixing."""
  for i, l in enumerate(cfg_dict["layers"]):
    H = l["mixer"]["heads"]
    t[f"l{i}.mix.rel"].zero_()
    t[f"l{i}.mix.pb"].zero_()
    t[f"l{i}.mix.talk"].copy_(torch.eye(H))
  return t


@pytest.mark.parametrize("mechanism", ["plain", "distance_bias", "head_bias", "talk", "softcap", "value_mix", "feed_forward", "qk_norm_weight", "all"])
def test_each_mechanism_alone(mechanism):
  on = lambda name: mechanism in (name, "all")
  cfg = model([layer(ff=40 if on("feed_forward") else 0, v_mix=on("value_mix"), softcap=1.5 if on("softcap") else 0.0, window=6),
               layer(ff=0, v_mix=on("value_mix"), softcap=1.5 if on("softcap") else 0.0, window=6)])
  full = ref.random_model(cfg, seed=11)
  t = _neutral(copy.deepcopy(full), cfg)
  for i in range(2):
    if on("distance_bias"):
      t[f"l{i}.mix.rel"] = full[f"l{i}.mix.rel"] * 3
    if on("head_bias"):
      t[f"l{i}.mix.pb"] = full[f"l{i}.mix.pb"]
    if on("talk"):
      t[f"l{i}.mix.talk"] = full[f"l{i}.mix.talk"]
    if not on("qk_norm_weight"):
      t[f"l{i}.mix.q.norm"].fill_(1.0)
      t[f"l{i}.mix.k.norm"].fill_(1.0)
    if on("softcap"):  # scores large enough for the cap to bend them
      t[f"l{i}.mix.q.norm"] = t[f"l{i}.mix.q.norm"] * 3
  toks = tokens_for(cfg, 19)
  want = ref.KifusunRef(cfg, t).forward(toks)
  engine, _ = make_engine(cfg, t)
  assert rel_err(whole(engine, toks), want) < 2e-5


def test_mechanism_functions_of_the_oracle_agree_with_closed_forms():
  # the oracle's own pieces against hand-computable cases (so a shared misreading cannot hide in both)
  assert ref.distance_bucket(3, 10, 40.0) == 3 and ref.distance_bucket(5, 10, 40.0) == 5 and ref.distance_bucket(39, 10, 40.0) == 9
  assert ref.distance_bucket(1000, 10, 40.0) == 9
  y = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
  assert torch.allclose(ref.unit_rms(y, 0.0), y / math.sqrt(12.5))
  assert abs(float(ref.gelu_tanh(torch.tensor(1.0, dtype=torch.float64))) - 0.8411919906082768) < 1e-12


# ---- schedules: the logits of a position do not depend on how it got there --------------------------------------------------------

def test_prefill_equals_token_by_token_decoding():
  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=1)
  toks = tokens_for(cfg, 30)
  want = ref.KifusunRef(cfg, t).forward(toks)
  engine, _ = make_engine(cfg, t)
  assert rel_err(whole(engine, toks), want) < 2e-5
  rows = [engine.step([(1, [tok], [0])]).cpu().double() for tok in toks]
  engine.release_pages(1)
  assert rel_err(torch.cat(rows), want) < 2e-5


@pytest.mark.parametrize("sizes", [[2, 2, 2, 3, 5, 16], [7, 1, 1, 2, 19], [1, 29], [13, 17]])
def test_portions_of_any_size(sizes):
  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=2)
  toks = tokens_for(cfg, sum(sizes))
  want = ref.KifusunRef(cfg, t).forward(toks)
  engine, _ = make_engine(cfg, t, tokens_per_page=8)
  got, at = [], 0
  for n in sizes:
    got.append(engine.step([(2, toks[at : at + n], list(range(n)))]).cpu().double())
    at += n
  assert rel_err(torch.cat(got), want) < 2e-5


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 2e-2)])
def test_a_step_longer_than_the_engine_takes_at_once_runs_in_slices(dtype, tol):
  """max_step_rows = 10: a 37-token portion beside a 5-token one is cut into four device steps, inside both runs."""
  cfg = model([layer(dim=32, vdim=16, window=9), layer(dim=32, vdim=16, window=20, ff=0)])
  t = ref.random_model(cfg, seed=8)
  oracle = ref.KifusunRef(cfg, t)
  a, b = tokens_for(cfg, 37, seed=1), tokens_for(cfg, 5, seed=2)
  engine, _ = make_engine(cfg, t, dtype=dtype, tokens_per_page=8, max_step_rows=10)
  got = engine.step([(0, a, list(range(37))), (3, b, [0, 4])]).cpu().double()
  want = torch.cat([oracle.forward(a), oracle.forward(b)[[0, 4]]])
  assert (rel_err(got, want) if dtype == "float32" else _rms_err(got, want)) < tol


def test_unequal_requests_in_one_batch_equal_each_alone_and_freed_pages_are_reused():
  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=3)
  oracle = ref.KifusunRef(cfg, t)
  lens = {"a": 23, "b": 9, "c": 1, "d": 14, "e": 17, "f": 6}
  toks = {k: tokens_for(cfg, n, seed=ord(k)) for k, n in lens.items()}
  want = {k: oracle.forward(v) for k, v in toks.items()}
  # a pool of 19 usable pages of 4 tokens: a + b + c + d need 6 + 3 + 1 + 4; e and f only fit into pages that were given back
  engine, _ = make_engine(cfg, t, tokens_per_page=4, num_pages=20, max_len=64)
  got = {k: [] for k in toks}
  at = {k: 0 for k in toks}
  slot_of = {"a": 0, "b": 1, "c": 2, "d": 3}
  plan = [  # (request, tokens in this step)
      [("a", 5), ("b", 2), ("c", 1), ("d", 3)],
      [("a", 1), ("b", 7), ("d", 1)],
      [("a", 9), ("d", 10)],
      [("a", 1), ("e", 4), ("f", 2)],  # e, f take the slots and pages of b, c
      [("a", 7), ("e", 1), ("f", 4)],
      [("e", 12)],
  ]
  used_pages = set()
  for step in plan:
    for k, _ in step:
      if k not in slot_of:
        done = [r for r, s in slot_of.items() if at[r] == lens[r]]
        slot_of[k] = slot_of.pop(done[0])
    entries = []
    for k, n in step:
      entries.append((slot_of[k], toks[k][at[k] : at[k] + n], list(range(n))))
    out = engine.step(entries).cpu().double()
    ps = engine.page_state
    for k, n in step:
      got[k].append(out[:n])
      out = out[n:]
      at[k] += n
      used_pages.update(ps.page_map[slot_of[k], : ps.num_pages_used[slot_of[k]]].tolist())
      if at[k] == lens[k]:
        engine.release_pages(slot_of[k])
  assert 0 not in used_pages and max(used_pages) <= 19
  for k in toks:
    assert at[k] == lens[k]
    assert rel_err(torch.cat(got[k]), want[k]) < 2e-5, k


def test_pool_exhaustion_is_an_error_not_a_wrong_answer():
  cfg = DEFAULT()
  engine, _ = make_engine(cfg, ref.random_model(cfg, seed=3), tokens_per_page=4, num_pages=5, max_len=64)
  engine.step([(0, tokens_for(cfg, 12), [])])
  with pytest.raises(ValueError, match="page pool"):
    engine.step([(1, tokens_for(cfg, 9), [])])


def test_long_decoding_across_many_pages_and_windows():
  cfg = model([layer(window=9), layer(window=4, ff=0)])
  t = ref.random_model(cfg, seed=4)
  toks = tokens_for(cfg, 70)
  want = ref.KifusunRef(cfg, t).forward(toks)
  engine, _ = make_engine(cfg, t, tokens_per_page=4, num_pages=24, max_len=96)
  first = engine.step([(3, toks[:6], list(range(6)))]).cpu().double()
  rows = [engine.step([(3, [tok], [0])]).cpu().double() for tok in toks[6:]]
  assert rel_err(torch.cat([first] + rows), want) < 2e-5


# ---- keys at the edges -----------------------------------------------------------------------------------------------------------

def _spiked(cfg, rows):
  """Weights under which ONLY keys in the last distance bucket count: the head bias shuts every key (sigmoid(-30)), the last row
  of the distance table opens it again.  With `far` = window - 1 that bucket is the last few distances inside the window (and
  everything beyond it): a window that is one key short loses an open key, one that is one key long gains one, and either changes
  the output by a large fraction instead of hiding among dozens of ordinary weights."""
  t = ref.random_model(cfg, seed=6, bias_rows=rows)
  for i in range(len(cfg["layers"])):
    t[f"l{i}.mix.pb"].fill_(-30.0)
    t[f"l{i}.mix.rel"].zero_()
    t[f"l{i}.mix.rel"][rows - 1].fill_(30.0)
  return t


@pytest.mark.parametrize("window,tokens_per_page", [(8, 4), (9, 8), (17, 16), (33, 16)])
def test_key_just_inside_and_just_outside_the_window(window, tokens_per_page):
  rows = 12
  cfg = model([layer(window=window, bias_max=float(window - 1), ff=0), layer(window=window, bias_max=float(window - 1))])
  t = _spiked(cfg, rows)
  assert ref.distance_bucket(window - 1, rows, window - 1.0) == rows - 1 and ref.distance_bucket(window // 2, rows, window - 1.0) < rows - 1
  toks = tokens_for(cfg, 3 * window + 3)
  oracle = ref.KifusunRef(cfg, t)
  want = oracle.forward(toks)
  # the same model with a window one key wider or narrower differs visibly: the test would see an off-by-one
  for other in (window - 1, window + 1):
    c2 = copy.deepcopy(cfg)
    for l in c2["layers"]:
      l["mixer"]["mask"]["size"] = other
    assert rel_err(ref.KifusunRef(c2, t).forward(toks), want) > 1e-2
  engine, _ = make_engine(cfg, t, tokens_per_page=tokens_per_page, num_pages=40, max_len=160)
  assert rel_err(whole(engine, toks), want) < 2e-5
  # and decoded one by one after a prompt that ends right at / before / after the window's and a page's edge
  for cut in (window - 1, window, window + 1, tokens_per_page, 2 * tokens_per_page + 1):
    head = engine.step([(1, toks[:cut], list(range(cut)))]).cpu().double()
    rows_out = [engine.step([(1, [tok], [0])]).cpu().double() for tok in toks[cut:]]
    engine.release_pages(1)
    assert rel_err(torch.cat([head] + rows_out), want) < 2e-5, cut


def test_a_far_key_among_many_is_found():
  """One key far back (window 150) matches the query of the last position exactly and is the only open one."""
  window, n = 150, 180
  cfg = model([layer(window=window, heads=2, kv_heads=1, dim=16, vdim=8, ff=0, softcap=0.0, bias_max=200.0, scale=1.0)], width=32)
  t = ref.random_model(cfg, seed=7)
  t["l0.mix.rel"].zero_()
  t["l0.mix.talk"].copy_(torch.eye(2))
  t["l0.mix.pb"].fill_(-12.0)  # a key opens only with a score near +12 or above: |q| |k| cos = 16 for parallel unit-RMS vectors
  toks = tokens_for(cfg, n, seed=8)
  oracle = ref.KifusunRef(cfg, t)
  want = oracle.forward(toks)
  engine, _ = make_engine(cfg, t, tokens_per_page=16, num_pages=16, max_len=200)
  got = whole(engine, toks)
  assert rel_err(got, want) < 2e-5
  # the test has teeth: some (query, key) pair at a distance beyond 100 carries real weight
  x = oracle.embed(toks)
  q, k, v, _ = oracle.qkv(0, x, None)
  w = ref.window_weights(q, k, oracle.t["l0.mix.rel"], oracle.t["l0.mix.pb"], oracle.t["l0.mix.talk"], 1.0, 0.0, window, 200.0,
                         torch.arange(n), torch.arange(n))
  far = torch.tril(torch.ones(n, n), diagonal=-100)  # pairs (i, j) with i - j >= 100 (w is zero beyond the window already)
  assert float((w.abs() * far).max()) > 1e-3


def test_first_tokens_of_a_sequence():
  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=9)
  oracle = ref.KifusunRef(cfg, t)
  engine, _ = make_engine(cfg, t)
  for n in (1, 2, 3):
    toks = tokens_for(cfg, n, seed=n)
    assert rel_err(whole(engine, toks), oracle.forward(toks)) < 2e-5


# ---- other sizes -------------------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("case", ["odd_sizes", "one_kv_head", "all_kv_heads", "window_one", "window_longer_than_sequence",
                                  "layers_differ", "mixing_starts_late", "no_mixing", "wide"])
def test_other_sizes(case):
  L = layer
  cfgs = {
      "odd_sizes": model([L(heads=6, kv_heads=3, dim=20, vdim=12, window=5, ff=36), L(heads=6, kv_heads=3, dim=20, vdim=12, window=3, ff=0)], width=72, vocab=53),
      "one_kv_head": model([L(heads=4, kv_heads=1, dim=8, vdim=8, window=6)], width=24),
      "all_kv_heads": model([L(heads=3, kv_heads=3, dim=16, vdim=4, window=6), L(heads=3, kv_heads=3, dim=16, vdim=4, window=6)], width=40),
      "window_one": model([L(window=1), L(window=1, ff=0)]),
      "window_longer_than_sequence": model([L(window=500, bias_max=600.0)]),
      "layers_differ": model([L(heads=2, kv_heads=2, dim=8, vdim=16, window=4, ff=24), L(heads=8, kv_heads=4, dim=12, vdim=8, window=11, ff=0, v_mix=False),
                              L(heads=4, kv_heads=2, dim=32, vdim=16, window=2, ff=56, softcap=0.0)], width=56),
      "mixing_starts_late": model([L(v_mix=False), L(v_mix=True), L(v_mix=False, ff=0), L(v_mix=True)]),
      "no_mixing": model([L(v_mix=False), L(v_mix=False)]),
      "wide": model([L(heads=8, kv_heads=2, dim=64, vdim=64, window=40, ff=192), L(heads=8, kv_heads=2, dim=64, vdim=64, window=24, ff=192)], width=128, vocab=300),
  }
  cfg = cfgs[case]
  t = ref.random_model(cfg, seed=13, bias_rows=7 if case == "odd_sizes" else 12)
  toks = tokens_for(cfg, 45)
  want = ref.KifusunRef(cfg, t).forward(toks)
  engine, _ = make_engine(cfg, t, tokens_per_page=8, num_pages=12)
  assert rel_err(whole(engine, toks), want) < 2e-5
  head = engine.step([(2, toks[:11], list(range(11)))]).cpu().double()
  tail = [engine.step([(2, [tok], [0])]).cpu().double() for tok in toks[11:]]
  assert rel_err(torch.cat([head] + tail), want) < 2e-5


# ---- bfloat16: the serving precision ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("case", ["small", "tiles"])
def test_bfloat16_engine_is_within_rounding_of_the_exact_model(case):
  if case == "small":
    cfg = DEFAULT()
  else:  # whole 128 x 64 tiles: the projections run on the tcgen05 GEMMs, the mixer on its tensor-core kernel
    cfg = model([layer(heads=4, kv_heads=2, dim=64, vdim=64, window=48, ff=256), layer(heads=4, kv_heads=2, dim=64, vdim=64, window=20, ff=256)],
                width=128, vocab=256)
  t = ref.random_model(cfg, seed=21)
  toks = tokens_for(cfg, 150 if case == "tiles" else 40)
  want = ref.KifusunRef(cfg, t).forward(toks)
  engine, _ = make_engine(cfg, t, dtype="bfloat16", tokens_per_page=16, num_pages=24, max_len=256)
  got = whole(engine, toks)
  rms = lambda a: float(a.pow(2).mean().sqrt())
  assert rms(got - want) / rms(want) < 2e-2
  # schedule independence holds in bf16 too, beyond rounding
  parts = [engine.step([(1, toks[:37], list(range(37)))]).cpu().double()]
  parts += [engine.step([(1, [tok], [0])]).cpu().double() for tok in toks[37:]]
  assert rms(torch.cat(parts) - want) / rms(want) < 2e-2


# ---- the framework's entry point: scheduler, sampler -------------------------------------------------------------------------------

def test_greedy_generation_through_the_offline_engine():
  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=17)
  oracle = ref.KifusunRef(cfg, t)
  config = pyconfig.from_model_dict(cfg, dtype="float32", per_device_batch_size=2, max_target_length=64, pagedattn_tokens_per_page=4,
                                    pagedattn_num_pages=30, decode_sampling_strategy="greedy")
  eng = offline_engine.OfflineEngine(config, params=t)
  prompts = [tokens_for(cfg, n, seed=30 + n) for n in (5, 11, 3, 8, 2)]  # five prompts over two slots: slots and pages are reused
  outs = eng.batch_inference(prompts, max_decode_length=9)
  for prompt, out in zip(prompts, outs):
    seq = list(prompt)
    for _ in range(9):
      logits = oracle.forward(seq)[-1]
      top2 = torch.topk(logits, 2).values
      assert float(top2[0] - top2[1]) > 1e-4, "near-tie in the test's own model; change the seed"
      seq.append(int(logits.argmax()))
    assert out.token_ids.tolist() == seq[len(prompt):]


# ---- the tensor-core mixer (bf16, head sizes in multiples of 16) ---------------------------------------------------------------------

def _rms_err(got, want):
  rms = lambda a: float(a.pow(2).mean().sqrt())
  return rms(got - want) / rms(want)


@pytest.mark.parametrize("heads,kv_heads,dim,vdim,window,page", [
    (4, 2, 32, 16, 5, 4), (8, 8, 16, 48, 33, 16), (16, 4, 64, 64, 100, 8), (12, 3, 48, 32, 20, 4), (2, 1, 128, 128, 70, 16),
    (1, 1, 16, 256, 9, 4), (4, 1, 96, 48, 40, 8),
    # heads too large for 64-key tiles: 32-key tiles, two warps per key group with half the heads each (8 + 8, and 3 + 3)
    (16, 4, 128, 128, 70, 16), (6, 6, 256, 64, 40, 8)])
def test_tensor_core_mixer_shapes_and_schedules(heads, kv_heads, dim, vdim, window, page):
  cfg = model([layer(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, window=window, ff=0, bias_max=float(window + 3)),
               layer(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, window=max(2, window // 2), ff=48)], width=64, vocab=90)
  t = ref.random_model(cfg, seed=23)
  oracle = ref.KifusunRef(cfg, t)
  toks = {k: tokens_for(cfg, n, seed=n) for k, n in (("a", 131), ("b", 37), ("c", 18))}
  want = {k: oracle.forward(v) for k, v in toks.items()}
  engine, _ = make_engine(cfg, t, dtype="bfloat16", tokens_per_page=page, num_pages=200 // page * 2, max_len=200)
  for k in toks:  # whole prompts: query tiles of 16 rows, the last one ragged
    assert _rms_err(whole(engine, toks[k]), want[k]) < 2e-2, k
  # a mixed batch: portions of a and b beside single tokens of c, then everything decoded token by token
  got = {k: [] for k in toks}
  at = {k: 0 for k in toks}
  slot = {"a": 0, "b": 1, "c": 2}
  for sizes in ({"a": 50, "b": 3, "c": 1}, {"a": 17, "b": 20, "c": 1}, {"a": 33, "c": 1}):
    entries = [(slot[k], toks[k][at[k] : at[k] + n], list(range(n))) for k, n in sizes.items()]
    out = engine.step(entries).cpu().double()
    for k, n in sizes.items():
      got[k].append(out[:n])
      out = out[n:]
      at[k] += n
  while any(at[k] < len(toks[k]) for k in toks):
    live = [k for k in toks if at[k] < len(toks[k])]
    out = engine.step([(slot[k], [toks[k][at[k]]], [0]) for k in live]).cpu().double()
    for i, k in enumerate(live):
      got[k].append(out[i : i + 1])
      at[k] += 1
  for k in toks:
    assert _rms_err(torch.cat(got[k]), want[k]) < 2e-2, k


@pytest.mark.parametrize("window,page", [(16, 8), (17, 4), (33, 16), (64, 16), (65, 64)])
def test_tensor_core_mixer_window_edges(window, page):
  rows = 24 if window > 40 else 12  # (more rows in the distance table: a narrower last bucket, fewer open keys)
  cfg = model([layer(heads=4, kv_heads=2, dim=32, vdim=16, window=window, bias_max=float(window - 1), ff=0),
               layer(heads=4, kv_heads=2, dim=32, vdim=16, window=window, bias_max=float(window - 1))])
  t = _spiked(cfg, rows)
  toks = tokens_for(cfg, 2 * window + 21)
  want = ref.KifusunRef(cfg, t).forward(toks)
  for other in (window - 1, window + 1):  # an off-by-one window would be far outside the tolerance below
    c2 = copy.deepcopy(cfg)
    for l in c2["layers"]:
      l["mixer"]["mask"]["size"] = other
    assert _rms_err(ref.KifusunRef(c2, t).forward(toks), want) > 8e-2
  engine, _ = make_engine(cfg, t, dtype="bfloat16", tokens_per_page=page, num_pages=600 // page, max_len=256)
  assert _rms_err(whole(engine, toks), want) < 2e-2
  for cut in (window - 1, window, window + 1, 16, 17):
    head = engine.step([(1, toks[:cut], list(range(cut)))]).cpu().double()
    tail = [engine.step([(1, [tok], [0])]).cpu().double() for tok in toks[cut:]]
    engine.release_pages(1)
    assert _rms_err(torch.cat([head] + tail), want) < 2e-2, cut


@pytest.mark.parametrize("heads,kv_heads,dim,vdim,window,page", [(8, 2, 64, 32, 150, 16), (6, 6, 32, 48, 97, 8), (16, 2, 16, 16, 260, 64)])
def test_decode_mixer_key_splits_and_long_windows(heads, kv_heads, dim, vdim, window, page):
  """Steps of single tokens only: the decode arm, windows of many 16-key tiles (several key splits, a ring of staged tiles that
  wraps), three sequences of unequal length, one key far back made to dominate."""
  cfg = model([layer(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, window=window, ff=0, bias_max=float(window)),
               layer(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, window=window - 40, ff=32)], width=64, vocab=90)
  t = ref.random_model(cfg, seed=31)
  oracle = ref.KifusunRef(cfg, t)
  lens = {"a": window + 90, "b": window - 3, "c": 21}
  toks = {k: tokens_for(cfg, n, seed=n) for k, n in lens.items()}
  want = {k: oracle.forward(v) for k, v in toks.items()}
  engine, _ = make_engine(cfg, t, dtype="bfloat16", tokens_per_page=page, num_pages=3 * ((window + 90 + page - 1) // page) + 2, max_len=window + 100)
  slot = {"a": 0, "b": 1, "c": 2}
  got = {k: [] for k in toks}
  for step in range(max(lens.values())):
    live = [k for k in toks if step < lens[k]]
    out = engine.step([(slot[k], [toks[k][step]], [0]) for k in live]).cpu().double()
    for i, k in enumerate(live):
      got[k].append(out[i : i + 1])
  for k in toks:
    assert _rms_err(torch.cat(got[k]), want[k]) < 2e-2, k
