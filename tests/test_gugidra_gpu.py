"""The Gugidra design on the layered engine against the plain restatement in oracle/gugidra_ref.py (numpy float64, same weights).

Small configurations with random weights; where random weights would hide a fault (a far key among hundreds, a state that is
lost or not reset) the weights are made so that it shows.  float32 engines are compared tightly, bfloat16 ones within rounding.
"""

import copy

import numpy as np
import pytest
import torch

from maxtext_indextts2_b200 import gugidra as g
from maxtext_indextts2_b200 import maxengine, offline_engine, pyconfig
from oracle import gugidra_ref as ref

pytestmark = pytest.mark.gpu

TIGHT = 3e-5


def as_torch(t):
  return {k: torch.from_numpy(np.asarray(v)).to(torch.bfloat16) for k, v in t.items()}


def make_engine(cfg_dict, tensors, dtype="float32", slots=4, tokens_per_page=4, num_pages=60, max_len=200, **kw):
  config = pyconfig.from_model_dict(cfg_dict, dtype=dtype, per_device_batch_size=slots, max_target_length=max_len,
                                    pagedattn_tokens_per_page=tokens_per_page, pagedattn_num_pages=num_pages, **kw)
  engine = maxengine.MaxEngine(config)
  engine.load_params(as_torch(tensors))
  engine.init_decode_state()
  return engine


def tokens_for(cfg_dict, n, seed=5):
  return np.random.Generator(np.random.PCG64(seed)).integers(0, cfg_dict["vocab"], size=n).tolist()


def rel_err(got, want):
  got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
  return float(np.abs(got - want).max() / np.abs(want).max())


def rms_err(got, want):
  got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
  return float(np.sqrt(((got - want) ** 2).mean()) / np.sqrt((want**2).mean()))


def whole(engine, toks, slot=0):
  out = engine.step([(slot, toks, list(range(len(toks))))]).cpu().numpy()
  engine.release_pages(slot)
  return out


def par(mlp=None, **kw):
  args = dict(heads=4, kv_heads=2, dim=24, r_heads=3, r_dim=12, r_vdim=20, rot_dims=16, rot_base=100.0, gate_cap=6.0, left_scale=1.3, right_scale=0.7)
  args.update(kw)
  return g.parallel_layer(mlp=mlp, **args)


def gla(mlp=None, **kw):
  args = dict(heads=3, dim=12, vdim=20, tau=4.0)
  args.update(kw)
  return g.gla_layer(mlp=mlp, **args)


def model(layers, width=40, vocab=61, loop=None, softcap=4.0, embed_scale=1.7):
  return g.model_dict(width, vocab, layers, eps=1e-5, embed_scale=embed_scale, logit_softcap=softcap, loop=loop)


MOE = lambda **kw: g.moe_ff(**{**dict(experts=6, top=2, ff=24, groups=3, keep=2, limit=1.0, shared_ff=16, shared_limit=1.5), **kw})
DEFAULT = lambda: model([par(g.dense_ff(56, 2.0)), gla(MOE()), par(MOE()), gla(g.dense_ff(32, 1.0))], loop={"start": 1, "stop": 3, "times": 2})


# ---- each mechanism alone ------------------------------------------------------------------------------------------------------

CASES = {
    "gla": lambda: model([gla()]),
    "softmax_attention": lambda: model([par(right_scale=0.0)]),
    "attention_all_channels_rotated": lambda: model([par(right_scale=0.0, rot_dims=24)]),
    "attention_no_rotation": lambda: model([par(right_scale=0.0, rot_dims=0)]),
    "mlstm": lambda: model([par(left_scale=0.0)]),
    "parallel_sum": lambda: model([par()]),
    "dense_ff": lambda: model([gla(g.dense_ff(56, 0.8))]),
    "dense_ff_wide_limit": lambda: model([gla(g.dense_ff(56, 50.0))]),
    "moe_no_groups": lambda: model([gla(MOE(groups=1, keep=1, shared_ff=0))]),
    "moe_groups": lambda: model([gla(MOE(experts=12, top=3, groups=4, keep=2, shared_ff=0))]),
    "moe_shared": lambda: model([gla(MOE())]),
    "moe_top_one": lambda: model([gla(MOE(top=1))]),
    "loop": lambda: model([gla(), par(), gla()], loop={"start": 1, "stop": 3, "times": 3}),
    "loop_from_layer_zero": lambda: model([gla(g.dense_ff(24, 2.0)), par()], loop={"start": 0, "stop": 2, "times": 2}),
    "loop_once": lambda: model([gla(), par()], loop={"start": 0, "stop": 1, "times": 1}),
    "no_softcap": lambda: model([par(g.dense_ff(24, 2.0))], softcap=0.0),
}


@pytest.mark.parametrize("case", sorted(CASES))
def test_each_mechanism_alone(case):
  cfg = CASES[case]()
  t = ref.random_model(cfg, seed=11)
  toks = tokens_for(cfg, 37)
  want = ref.logits_of(cfg, t, toks)
  engine = make_engine(cfg, t)
  assert rel_err(whole(engine, toks), want) < TIGHT


def test_mechanism_functions_of_the_oracle_agree_with_closed_forms():
  # the oracle's own pieces against hand-computable cases (so a shared misreading cannot hide in both)
  t = np.array([[[1.0, 0.0, 2.0, 5.0]]])
  r = ref.rotate_pairs(t, np.array([1]), 2, 10.0)  # one pair, angle 1 * 10^0 = 1 radian; channels 2, 3 pass
  assert np.allclose(r[0, 0], [np.cos(1.0), np.sin(1.0), 2.0, 5.0])
  assert np.allclose(ref.clamped_gate(np.array([3.0]), np.array([-9.0]), 2.0), 2.0 / (1 + np.exp(-3.404)) * (-2.0 + 1.0))
  # routing: 6 experts in 3 groups, 2 groups kept; the correction steers the choice, the weights ignore it
  logits = np.log(np.array([[0.9, 0.1, 0.5, 0.6, 0.8, 0.7]]) / (1 - np.array([[0.9, 0.1, 0.5, 0.6, 0.8, 0.7]])))
  chosen, w = ref.route(logits, np.eye(6), np.array([0.0, 0.0, 0.0, 0.0, -0.55, 0.0]), 2, 3, 2)
  # groups' scores: 1.0, 1.1, 0.25 + 0.7 = 0.95 -> groups 1 and 0; best two choice scores among their experts: 0.9 (e0), 0.6 (e3);
  # without the correction group 2 (1.5) and its expert 4 (0.8) would have won
  assert chosen.tolist() == [[0, 3]] and np.allclose(w, [[0.9 / 1.5, 0.6 / 1.5]])
  # mLSTM, first token: m = max(f + 0, i); with i very negative the floor exp(-m) of the denominator rules
  S, n, m = np.zeros((1, 1, 1)), np.zeros((1, 1)), np.zeros(1)
  o = ref.mlstm_scan(np.array([[[2.0]]]), np.array([[[3.0]]]), np.array([[[5.0]]]), np.array([[-4.0]]), np.array([[-1.0]]), S, n, m)
  assert np.isclose(m[0], -1.0) and np.isclose(S[0, 0, 0], np.exp(-3.0) * 15.0)
  assert np.isclose(o[0, 0, 0], np.exp(-3.0) * 30.0 / (max(np.exp(-3.0) * 6.0, np.exp(1.0)) + 1e-6))
  S = np.zeros((1, 1, 1))
  o = ref.gla_scan(np.ones((2, 1, 1)), np.ones((2, 1, 1)), np.array([[[1.0]], [[10.0]]]), np.full((2, 1, 1), 0.5), S)
  assert o[:, 0, 0].tolist() == [1.0, 10.5]


# ---- schedules: the logits of a position do not depend on how it got there --------------------------------------------------------

def test_prefill_equals_token_by_token_decoding():
  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=1)
  toks = tokens_for(cfg, 45)
  want = ref.logits_of(cfg, t, toks)
  engine = make_engine(cfg, t)
  first = whole(engine, toks)
  assert rel_err(first, want) < TIGHT
  rows = [engine.step([(1, [tok], [0])]).cpu().numpy() for tok in toks]
  engine.release_pages(1)
  assert rel_err(np.concatenate(rows), want) < TIGHT
  assert np.array_equal(np.concatenate(rows), first)  # float32: the same bits whatever the cut


@pytest.mark.parametrize("sizes", [[2, 2, 2, 3, 5, 16, 17, 15], [7, 1, 1, 2, 33, 18], [1, 61], [16, 16, 30], [31, 31]])
def test_portions_of_any_size(sizes):
  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=2)
  toks = tokens_for(cfg, sum(sizes))
  want = ref.logits_of(cfg, t, toks)
  engine = make_engine(cfg, t, tokens_per_page=8)
  got, at = [], 0
  for n in sizes:
    got.append(engine.step([(2, toks[at : at + n], list(range(n)))]).cpu().numpy())
    at += n
  assert rel_err(np.concatenate(got), want) < TIGHT


@pytest.mark.parametrize("dtype,tol", [("float32", TIGHT), ("bfloat16", 3e-2)])
def test_a_step_longer_than_the_engine_takes_at_once_runs_in_slices(dtype, tol):
  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=4)
  toks = {0: tokens_for(cfg, 50, seed=1), 1: tokens_for(cfg, 27, seed=2)}
  engine = make_engine(cfg, t, dtype=dtype, max_step_rows=19)  # slices cut both runs; the recurrent state crosses the cuts
  out = engine.step([(s, v, list(range(len(v)))) for s, v in toks.items()]).cpu().numpy()
  want = np.concatenate([ref.logits_of(cfg, t, v) for v in toks.values()])
  assert rms_err(out, want) < tol


def test_unequal_requests_in_one_batch_equal_each_alone_and_freed_slots_and_pages_are_reused():
  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=3)
  lens = {"a": 43, "b": 9, "c": 1, "d": 14, "e": 37, "f": 6}
  toks = {k: tokens_for(cfg, n, seed=ord(k)) for k, n in lens.items()}
  want = {k: ref.logits_of(cfg, t, v) for k, v in toks.items()}
  # 19 usable pages of 4 tokens: a + b + c + d take 11 + 3 + 1 + 4; e and f only fit into pages that were given back, and they
  # inherit state slots whose recurrent state b and c left behind
  engine = make_engine(cfg, t, tokens_per_page=4, num_pages=20, max_len=64)
  got, at = {k: [] for k in toks}, {k: 0 for k in toks}
  slot_of = {"a": 0, "b": 1, "c": 2, "d": 3}
  plan = [
      [("a", 5), ("b", 2), ("c", 1), ("d", 3)],
      [("a", 1), ("b", 7), ("d", 1)],
      [("a", 19), ("d", 10)],
      [("a", 1), ("e", 4), ("f", 2)],
      [("a", 17), ("e", 1), ("f", 4)],
      [("e", 32)],
  ]
  for step in plan:
    for k, _ in step:
      if k not in slot_of:
        done = [r for r, s in slot_of.items() if at[r] == lens[r]]
        slot_of[k] = slot_of.pop(done[0])
    out = engine.step([(slot_of[k], toks[k][at[k] : at[k] + n], list(range(n))) for k, n in step]).cpu().numpy()
    for k, n in step:
      got[k].append(out[:n])
      out = out[n:]
      at[k] += n
      if at[k] == lens[k]:
        engine.release_pages(slot_of[k])
  for k in toks:
    assert at[k] == lens[k]
    assert rel_err(np.concatenate(got[k]), want[k]) < TIGHT, k


def test_a_reused_slot_starts_from_zero_state_even_without_a_release_clearing_it():
  cfg = model([gla(), par()])
  t = ref.random_model(cfg, seed=8)
  engine = make_engine(cfg, t)
  a, b = tokens_for(cfg, 30, seed=1), tokens_for(cfg, 12, seed=2)
  engine.step([(0, a, [])])
  for st in engine._states:  # leave the first request's state (and some dirt) behind when the slot is handed on
    for s in st:
      s[0].add_(3.0)
  ps = engine.page_manager.release_pages(page_state=engine.page_state, page_group_id=0)
  engine.page_state = ps
  assert rel_err(engine.step([(0, b, list(range(12)))]).cpu().numpy(), ref.logits_of(cfg, t, b)) < TIGHT


def test_pool_exhaustion_is_an_error_not_a_wrong_answer():
  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=3)
  engine = make_engine(cfg, t, tokens_per_page=4, num_pages=5, max_len=64)
  engine.step([(0, tokens_for(cfg, 10), [9])])
  with pytest.raises(ValueError):
    engine.step([(1, tokens_for(cfg, 9), [8])])


def test_long_decoding_across_many_pages():
  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=6)
  toks = tokens_for(cfg, 150)
  want = ref.logits_of(cfg, t, toks)
  engine = make_engine(cfg, t, tokens_per_page=4, num_pages=50)
  got = [engine.step([(3, toks[:5], list(range(5)))]).cpu().numpy()]
  got += [engine.step([(3, [tok], [0])]).cpu().numpy() for tok in toks[5:]]
  assert rel_err(np.concatenate(got), want) < TIGHT


# ---- far keys, page borders, the first tokens ----------------------------------------------------------------------------------------

def _peaky(cfg, seed):
  """Attention whose scores spread widely, so that single keys (also far ones) carry most of a query's weight; a recurrence that
  forgets slowly, so that a token hundreds of steps back still matters."""
  t = ref.random_model(cfg, seed=seed)
  for i, l in enumerate(cfg["layers"]):
    if l["type"] == "parallel":
      t[f"l{i}.mix.left.q"] = t[f"l{i}.mix.left.q"] * 8.0
      t[f"l{i}.mix.right.f.b"] = t[f"l{i}.mix.right.f.b"] + 4.0
    else:
      t[f"l{i}.mix.a2.b"] = t[f"l{i}.mix.a2.b"] + 5.0
  return {k: ref.on_bf16_grid(v) for k, v in t.items()}


class _Blind(ref.GugidraRef):
  """The oracle with a fault: the attention cannot see keys further back than `reach`."""

  reach = 10**9

  def attention(self, i, h, pos, st):
    keep = ref.softmax_attention
    try:
      def near(q, k, v, q_pos, k_pos, scale):
        H, G = q.shape[1], k.shape[1]
        out = np.zeros((q.shape[0], H, v.shape[2]))
        for r in range(q.shape[0]):
          lo = max(0, int(q_pos[r]) - self.reach)
          out[r] = keep(q[r : r + 1], k[lo:], v[lo:], q_pos[r : r + 1], k_pos[lo:], scale)[0]
        return out
      ref.softmax_attention = near
      return super().attention(i, h, pos, st)
    finally:
      ref.softmax_attention = keep


@pytest.mark.parametrize("page", [4, 16, 64])
def test_far_keys_and_page_borders(page):
  cfg = model([par(), gla(), par(g.dense_ff(24, 2.0))], softcap=0.0)
  t = _peaky(cfg, seed=21)
  n = 330
  toks = tokens_for(cfg, n)
  want = ref.logits_of(cfg, t, toks)
  blind = _Blind(cfg, t)
  blind.reach = 300
  assert rms_err(blind.forward(toks, blind.new_state())[301:], want[301:]) > 1e-3  # losing keys 300 back would show
  engine = make_engine(cfg, t, tokens_per_page=page, num_pages=700 // page + 2, max_len=400)
  assert rel_err(whole(engine, toks), want) < TIGHT
  # a prompt that ends at, one before and one after a page border, then decoding across the next borders
  for cut in (2 * page - 1, 2 * page, 2 * page + 1):
    got = [engine.step([(1, toks[:cut], list(range(cut)))]).cpu().numpy()]
    got += [engine.step([(1, [tok], [0])]).cpu().numpy() for tok in toks[cut : cut + page + 3]]
    engine.release_pages(1)
    assert rel_err(np.concatenate(got), want[: cut + page + 3]) < TIGHT, cut
  # far keys seen from decoded tokens
  got = [engine.step([(2, toks[:310], [])]).cpu().numpy()] + [engine.step([(2, [tok], [0])]).cpu().numpy() for tok in toks[310:]]
  assert rel_err(np.concatenate(got[1:]), want[310:]) < TIGHT


def test_first_tokens_of_a_sequence():
  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=9)
  engine = make_engine(cfg, t)
  for n in (1, 2, 3):
    toks = tokens_for(cfg, n, seed=n)
    assert rel_err(whole(engine, toks), ref.logits_of(cfg, t, toks)) < TIGHT
  # input gates far below the forget path: the mLSTM's denominator sits on its floor exp(-m) at the first tokens
  low = copy.deepcopy(t)
  for i, l in enumerate(cfg["layers"]):
    if l["type"] == "parallel":
      low[f"l{i}.mix.right.i.b"] = ref.on_bf16_grid(low[f"l{i}.mix.right.i.b"] - 5.0)
  toks = tokens_for(cfg, 6, seed=7)
  engine = make_engine(cfg, low)
  assert rel_err(whole(engine, toks), ref.logits_of(cfg, low, toks)) < TIGHT


# ---- other sizes ------------------------------------------------------------------------------------------------------------------

SIZES = {
    "odd_width": lambda: model([par(g.dense_ff(30, 2.0)), gla(MOE())], width=36, vocab=47),
    "one_kv_head": lambda: model([par(kv_heads=1)]),
    "as_many_kv_heads_as_heads": lambda: model([par(kv_heads=4)]),
    "one_head_everywhere": lambda: model([par(heads=1, kv_heads=1, r_heads=1), gla(heads=1)]),
    "value_size_not_a_multiple_of_the_column_block": lambda: model([par(r_vdim=22), gla(vdim=18)]),
    "key_size_over_the_smallest_register_tile": lambda: model([par(r_dim=40), gla(dim=72, vdim=8)]),
    "wide_recurrent_heads": lambda: model([gla(heads=2, dim=136, vdim=40)], width=64),
    "big_attention_heads": lambda: model([par(heads=2, kv_heads=1, dim=72, rot_dims=40)], width=64),
    "attention_heads_beyond_the_default_shared_memory": lambda: model([par(heads=2, kv_heads=1, dim=160, rot_dims=64)], width=64),
    "widest_recurrent_heads": lambda: model([gla(heads=1, dim=256, vdim=16), par(heads=2, kv_heads=2, dim=16, r_heads=1, r_dim=200, r_vdim=24)], width=64),
    "groups_all_kept": lambda: model([gla(MOE(groups=3, keep=3))]),
    "one_expert_per_group": lambda: model([gla(MOE(experts=6, groups=6, keep=3, top=3))]),
    "every_expert_of_the_kept_groups": lambda: model([gla(MOE(experts=8, groups=4, keep=2, top=4))]),
    "many_experts": lambda: model([gla(MOE(experts=40, groups=8, keep=3, top=5, ff=8))]),
    "layers_without_feed_forward": lambda: model([par(), gla(), par()]),
    "loop_is_the_whole_model": lambda: model([par(MOE()), gla()], loop={"start": 0, "stop": 2, "times": 2}),
    "loop_at_the_end": lambda: model([gla(), par(g.dense_ff(24, 2.0))], loop={"start": 1, "stop": 2, "times": 3}),
    "embedding_scale_one": lambda: model([gla(g.dense_ff(24, 2.0))], embed_scale=1.0),
}


@pytest.mark.parametrize("case", sorted(SIZES))
def test_other_sizes(case):
  cfg = SIZES[case]()
  t = ref.random_model(cfg, seed=13)
  toks = tokens_for(cfg, 41)
  want = ref.logits_of(cfg, t, toks)
  engine = make_engine(cfg, t, tokens_per_page=8)
  got = [engine.step([(0, toks[:22], list(range(22)))]).cpu().numpy(), engine.step([(0, toks[22:39], list(range(17)))]).cpu().numpy()]
  got += [engine.step([(0, [tok], [0])]).cpu().numpy() for tok in toks[39:]]
  assert rel_err(np.concatenate(got), want) < TIGHT


@pytest.mark.parametrize("case", ["default", "tiles"])
def test_bfloat16_engine_is_within_rounding_of_the_exact_model(case):
  if case == "default":
    cfg = DEFAULT()
  else:  # sizes made of whole tiles of the tensor-core kernels
    cfg = model([par(g.dense_ff(128, 2.0), heads=4, kv_heads=2, dim=64, r_heads=2, r_dim=32, r_vdim=64, rot_dims=64),
                 gla(MOE(ff=64, shared_ff=64), heads=2, dim=32, vdim=64)], width=128, vocab=256, loop={"start": 0, "stop": 2, "times": 2})
  t = ref.random_model(cfg, seed=15)
  toks = tokens_for(cfg, 90)
  want = ref.logits_of(cfg, t, toks)
  engine = make_engine(cfg, t, dtype="bfloat16", tokens_per_page=16, num_pages=30)
  assert rms_err(whole(engine, toks), want) < 3e-2
  got = [engine.step([(1, toks[:70], list(range(70)))]).cpu().numpy()] + [engine.step([(1, [tok], [0])]).cpu().numpy() for tok in toks[70:]]
  assert rms_err(np.concatenate(got), want) < 3e-2


# ---- the tensor-core attention (bf16, head sizes in multiples of 16) ------------------------------------------------------------------

@pytest.mark.parametrize("heads,kv_heads,dim,page", [(4, 2, 64, 16), (2, 2, 16, 8), (8, 1, 32, 64), (6, 2, 48, 4), (5, 1, 96, 16), (4, 4, 128, 32), (2, 1, 256, 16)])
def test_tensor_core_attention_shapes_and_schedules(heads, kv_heads, dim, page):
  """Every head size of the tensor-core arm, one to eight query heads per key head (several CTAs per key head beyond four
  warps), prompts in portions that end inside, at and after the 64-key (32-key) tiles, 16-row query tiles that start anywhere,
  then single tokens; peaky scores so that single far keys matter."""
  cfg = model([par(heads=heads, kv_heads=kv_heads, dim=dim, rot_dims=dim // 2, r_heads=1, r_dim=16, r_vdim=16, right_scale=0.1),
               par(g.dense_ff(32, 2.0), heads=heads, kv_heads=kv_heads, dim=dim, rot_dims=dim, r_heads=1, r_dim=16, r_vdim=16)], width=64, vocab=90, softcap=0.0)
  t = _peaky(cfg, seed=dim + heads)
  n = 150
  toks = tokens_for(cfg, n, seed=dim)
  want = ref.logits_of(cfg, t, toks)
  engine = make_engine(cfg, t, dtype="bfloat16", tokens_per_page=page, num_pages=2 * (n // page + 2) + 2, max_len=n + 8)
  assert rms_err(whole(engine, toks), want) < 3e-2
  for cuts in ([63, 1, 1, 30, 33], [64, 64], [65, 5, 58, 9], [31, 2, 31, 33, 7, 25]):
    got, at = [], 0
    for c in cuts:
      got.append(engine.step([(1, toks[at : at + c], list(range(c)))]).cpu().numpy())
      at += c
    got += [engine.step([(1, [tok], [0])]).cpu().numpy() for tok in toks[at : at + 6]]
    engine.release_pages(1)
    assert rms_err(np.concatenate(got), want[: at + 6]) < 3e-2, cuts
  # two sequences side by side, one in the middle of its prompt, one decoding
  engine.step([(0, toks[:70], []), (2, toks[:101], [])])
  out = engine.step([(0, toks[70:90], list(range(20))), (2, [toks[101]], [0])]).cpu().numpy()
  assert rms_err(out, np.concatenate([want[70:90], want[101:102]])) < 3e-2


# ---- the framework's entry point: scheduler, sampler -------------------------------------------------------------------------------

def test_greedy_generation_through_the_offline_engine():
  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=17)
  config = pyconfig.from_model_dict(cfg, dtype="float32", per_device_batch_size=2, max_target_length=64, pagedattn_tokens_per_page=4,
                                    pagedattn_num_pages=30, decode_sampling_strategy="greedy")
  eng = offline_engine.OfflineEngine(config, params=as_torch(t))
  prompts = [tokens_for(cfg, n, seed=30 + n) for n in (5, 11, 3, 8, 2)]  # five prompts over two slots: slots, pages and state are reused
  outs = eng.batch_inference(prompts, max_decode_length=9)
  for prompt, out in zip(prompts, outs):
    seq = list(prompt)
    for _ in range(9):
      logits = ref.logits_of(cfg, t, seq)[-1]
      top2 = np.sort(logits)[-2:]
      assert float(top2[1] - top2[0]) > 1e-4, "near-tie in the test's own model; change the seed"
      seq.append(int(logits.argmax()))
    assert out.token_ids.tolist() == seq[len(prompt):]


# ---- the command line: a trace of batched steps replayed through bin/trace_run --------------------------------------------------------

@pytest.mark.parametrize("dtype,tol", [("float32", TIGHT), ("bfloat16", 5e-2)])  # (bfloat16: per step, some of few rows)
def test_trace_runner_replays_a_mixed_schedule(tmp_path, dtype, tol):
  import json
  import os
  import subprocess

  from tests.test_gugidra_host import _write_safetensors

  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=23)
  model_dir = tmp_path / "model"
  os.makedirs(model_dir)
  with open(model_dir / "config.json", "w") as f:
    json.dump(cfg, f)
  _write_safetensors(model_dir / "model.safetensors", as_torch(t))
  lens = {"a": 70, "b": 9, "c": 33, "d": 5, "e": 40, "f": 20}
  toks = {k: tokens_for(cfg, n, seed=ord(k)) for k, n in lens.items()}
  # four pages of 64 tokens: a, b, c fill them (2 + 1 + 1); d, e and f fit only into what b and c give back, and take their slots
  plan = [[("a", 30), ("b", 2)], [("a", 1), ("b", 7), ("c", 33)], [("a", 35), ("d", 2)], [("a", 1), ("d", 3), ("e", 39)], [("a", 3), ("e", 1), ("f", 20)]]
  at = {k: 0 for k in toks}
  lines, rows = [], []
  for n, step in enumerate(plan):
    entries, end = [], []
    for k, c in step:
      entries.append({"id": k, "tokens": toks[k][at[k] : at[k] + c], "want": list(range(c))})
      rows.append((n, k, at[k], c))
      at[k] += c
      if at[k] == lens[k]:
        end.append(k)
    lines.append(json.dumps({"step": n, "entries": entries, "end": end}))
  root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
  out_dir = tmp_path / "out"
  p = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(model_dir), "--dtype", dtype, "--out", str(out_dir), "--max-tokens", "256"],
                     input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
  assert p.returncode == 0, p.stderr[-2000:]
  assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {n}" for n in range(len(plan))]
  want = {k: ref.logits_of(cfg, t, v) for k, v in toks.items()}
  V = cfg["vocab"]
  errs = []
  for n in range(len(plan)):
    got = np.fromfile(out_dir / f"{n}.f32", dtype="<f4").reshape(-1, V)
    exp = np.concatenate([want[k][lo : lo + c] for s, k, lo, c in rows if s == n])
    assert got.shape == exp.shape
    errs.append(rms_err(got, exp))
  assert max(errs) < tol, errs
