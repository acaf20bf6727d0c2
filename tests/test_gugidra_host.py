"""Host-side pieces of the Gugidra design: config reading, checks, the plan of layer runs.  No GPU."""

import json
import os
import struct

import numpy as np
import pytest
import torch

from maxtext_indextts2_b200 import gugidra as g
from maxtext_indextts2_b200 import params as params_lib, pyconfig
from oracle import gugidra_ref as ref


def _write_safetensors(path, tensors):
  header, blobs, at = {}, [], 0
  for k, v in tensors.items():
    raw = v.contiguous().view(torch.uint8).numpy().tobytes()
    header[k] = {"dtype": "BF16", "shape": list(v.shape), "data_offsets": [at, at + len(raw)]}
    blobs.append(raw)
    at += len(raw)
  text = json.dumps(header).encode()
  with open(path, "wb") as f:
    f.write(struct.pack("<Q", len(text)) + text + b"".join(blobs))


def _model():
  moe = g.moe_ff(experts=6, top=2, ff=24, groups=3, keep=2, limit=1.0, shared_ff=16, shared_limit=1.5)
  layers = [g.parallel_layer(4, 2, 24, 3, 12, 20, mlp=g.dense_ff(56, 2.0), rot_dims=16, rot_base=100.0, left_scale=1.3, right_scale=0.7),
            g.gla_layer(3, 12, 20, tau=4.0, mlp=moe), g.gla_layer(2, 8, 12, mlp=None)]
  return g.model_dict(40, 61, layers, eps=1e-5, embed_scale=1.7, logit_softcap=4.0, loop={"start": 1, "stop": 3, "times": 2})


def test_layer_runs_unroll_the_loop():
  assert g.layer_runs(3, None) == [(0, -1, False), (1, -1, False), (2, -1, False)]
  assert g.layer_runs(4, {"start": 1, "stop": 3, "times": 2}) == [(0, -1, False), (1, 0, True), (2, 0, False), (1, 1, True), (2, 1, False), (3, -1, False)]
  assert g.layer_runs(2, {"start": 0, "stop": 2, "times": 1}) == [(0, 0, True), (1, 0, False)]
  assert [r[0] for r in ref.GugidraRef(_model(), ref.random_model(_model())).runs] == [0, 1, 2, 1, 2]


def test_model_folder_round_trip_and_plan(tmp_path):
  cfg = _model()
  tensors = {k: torch.from_numpy(v).to(torch.bfloat16) for k, v in ref.random_model(cfg, seed=1).items()}
  os.makedirs(tmp_path / "m")
  with open(tmp_path / "m" / "config.json", "w") as f:
    json.dump(cfg, f)
  _write_safetensors(tmp_path / "m" / "model.safetensors", tensors)
  loaded = params_lib.load_model_dir(str(tmp_path / "m"))
  assert set(loaded) == set(tensors) and all(torch.equal(loaded[k], v) for k, v in tensors.items())
  config = pyconfig.from_model_dir(str(tmp_path / "m"), per_device_batch_size=2, max_target_length=40, pagedattn_num_pages=9, pagedattn_tokens_per_page=8)
  assert config.decoder_block == "gugidra" and config.emb_dim == 40 and config.vocab_size == 61 and config.num_decoder_layers == 3
  assert config.embedding_scale == 1.7 and config.final_logits_soft_cap == 4.0 and config.layer_loop == {"start": 1, "stop": 3, "times": 2}
  plan = g.model_plan(config, loaded)
  runs = plan["layers"]
  assert [r["weights"] for r in runs] == [0, 1, 2, 1, 2]
  assert [r["add_embedding"] for r in runs] == [0, 0, 0, 1, 0] and [r["add_vector"] is not None for r in runs] == [False, True, False, True, False]
  assert torch.equal(runs[3]["add_vector"], tensors["loop.step"][1].float()) and runs[1]["w_in"] is runs[3]["w_in"]
  p0 = runs[0]
  assert p0["attn"]["values_are_keys"] == 1 and p0["attn"]["out_scale"] == 1.3 and p0["rec"]["out_scale"] == 0.7 and p0["rec"]["kind"] == "mlstm"
  n0 = 4 * 24 + 2 * 24 + 3 * 12 * 2 + 3 * 20 * 2 + 2 * 3
  assert p0["n_in"] == n0 and p0["w_in"].shape == (n0, 40) and p0["wo"].shape == (40, 4 * 24 + 3 * 20)  # (width 40: no padding to tiles)
  assert torch.equal(p0["w_in"][4 * 24 : 6 * 24], tensors["l0.mix.left.k"]) and torch.equal(p0["w_in"][-3:], tensors["l0.mix.right.f"])
  assert torch.equal(p0["b_in"][: 4 * 24], tensors["l0.mix.left.q.b"].float()) and float(p0["b_in"][6 * 24 :].abs().max()) == 0.0
  assert torch.allclose(p0["bo"], tensors["l0.mix.left.o.b"].float() * 1.3)
  assert p0["attn"]["rot_freq"].dtype == torch.float64
  assert torch.allclose(p0["attn"]["rot_freq"], torch.tensor([100.0 ** (-2.0 * i / 16) for i in range(8)], dtype=torch.float64), rtol=1e-14)
  assert torch.equal(p0["w_gate_up"][0::2], tensors["l0.mlp.gate"]) and torch.equal(p0["w_gate_up"][1::2], tensors["l0.mlp.up"])
  p1 = runs[1]
  assert p1["rec"]["kind"] == "gla" and p1["rec"]["decay_rank"] == 5 and p1["attn"] is None and p1["b_in"] is None
  assert torch.equal(p1["rec"]["decay_up_t"], tensors["l1.mix.a2"].float().t()) and p1["rec"]["out_norm"].shape == (60,)
  m = p1["moe"]
  assert (m["experts"], m["top"], m["groups"], m["keep_groups"], m["shared_ff"]) == (6, 2, 3, 2, 16) and m["w_gate_up"].shape == (6, 48, 40)
  assert torch.equal(m["w_gate_up"][4][1::2], tensors["l1.mlp.e4.up"]) and torch.equal(m["w_down"][5], tensors["l1.mlp.e5.down"])
  assert runs[2]["ff_kind"] == "none" and runs[2]["moe"] is None


def test_input_projection_is_padded_to_whole_tiles_when_the_width_allows():
  cfg = g.model_dict(64, 50, [g.gla_layer(2, 8, 16)])
  config = pyconfig.from_model_dict(cfg, per_device_batch_size=1, max_target_length=16, pagedattn_num_pages=4, pagedattn_tokens_per_page=8)
  t = g.random_tensors(config, seed=0)
  plan = g.model_plan(config, t)["layers"][0]
  n = 2 * 8 * 2 + 2 * 16 * 2 + 16
  assert plan["n_in"] == 128 and float(plan["w_in"][n:].float().abs().max()) == 0.0 and float(plan["w_in"][:n].float().abs().min()) >= 0.0


@pytest.mark.parametrize("break_it,match", [
    (lambda c: c["layers"][0].update(type="conv"), "mixer type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(vdim=8), "vdim must equal dim"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=30), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].update(tau=0.0), "tau"),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "feed-forward kind"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "do not fit together"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "do not fit together"),
    (lambda c: c["loop"].update(stop=7), "loop"),
    (lambda c: c.update(architecture="Other"), "architecture"),
])
def test_bad_configs_are_refused(break_it, match):
  cfg = _model()
  break_it(cfg)
  with pytest.raises(ValueError, match=match):
    pyconfig.from_model_dict(cfg, per_device_batch_size=1, max_target_length=16, pagedattn_num_pages=4, pagedattn_tokens_per_page=8)


def test_missing_or_misshaped_tensors_are_refused():
  cfg = _model()
  config = pyconfig.from_model_dict(cfg, per_device_batch_size=1, max_target_length=16, pagedattn_num_pages=4, pagedattn_tokens_per_page=8)
  t = {k: torch.from_numpy(v).to(torch.bfloat16) for k, v in ref.random_model(cfg, seed=1).items()}
  bad = dict(t)
  bad["l0.mix.right.norm"] = bad["l0.mix.right.norm"][:-1]
  with pytest.raises(ValueError, match="l0.mix.right.norm"):
    g.model_plan(config, bad)
  bad = dict(t)
  del bad["l1.mlp.e3.down"]
  with pytest.raises(KeyError):
    g.model_plan(config, bad)
