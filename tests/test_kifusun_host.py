"""Host-side pieces of the layered engine and of the Kifusun design: no GPU."""

import json
import os
import struct

import numpy as np
import pytest
import torch

from maxtext_indextts2_b200 import kifusun, page_manager, params as params_lib, pyconfig
from oracle import kifusun_ref as ref


def _model(layers, width=48, vocab=61):
  return {"architecture": "Kifusun", "vocab": vocab, "width": width, "embedding": {"scale": 2.5}, "norm": {"eps": 1e-6}, "layers": layers}


def _write_safetensors(path, tensors):
  header, blobs, at = {}, [], 0
  names = {torch.bfloat16: "BF16", torch.float32: "F32", torch.int32: "I32"}
  for k, v in tensors.items():
    raw = v.contiguous().view(torch.uint8).numpy().tobytes() if v.dim() else v.reshape(1).view(torch.uint8).numpy().tobytes()
    header[k] = {"dtype": names[v.dtype], "shape": list(v.shape), "data_offsets": [at, at + len(raw)]}
    blobs.append(raw)
    at += len(raw)
  text = json.dumps(header).encode()
  with open(path, "wb") as f:
    f.write(struct.pack("<Q", len(text)) + text + b"".join(blobs))


@pytest.mark.parametrize("rows,far,window", [(32, 100.0, 90), (10, 40.0, 64), (7, 33.0, 50), (12, 500.0, 700), (6, 9.0, 30)])
def test_distance_bucket_table_matches_the_rule(rows, far, window):
  table = kifusun.distance_bucket_table(window, rows, far)
  want = [ref.distance_bucket(n, rows, far) for n in range(window)]
  assert table.tolist() == want
  assert table.max() <= rows - 1 and (np.diff(table) >= 0).all()


def test_model_folder_round_trip(tmp_path):
  cfg = _model([kifusun.attention_layer(4, 2, 24, 16, 7, ff=40), kifusun.attention_layer(2, 1, 8, 4, 3, ff=0, v_mix=False)])
  tensors = ref.random_model(cfg, seed=1)
  tensors["table"] = torch.arange(6, dtype=torch.int32).reshape(2, 3)
  os.makedirs(tmp_path / "m")
  with open(tmp_path / "m" / "config.json", "w") as f:
    json.dump(cfg, f)
  _write_safetensors(tmp_path / "m" / "model.safetensors", tensors)
  loaded = params_lib.load_model_dir(str(tmp_path / "m"))
  assert set(loaded) == set(tensors)
  for k, v in tensors.items():
    assert loaded[k].dtype == v.dtype and loaded[k].shape == v.shape and torch.equal(loaded[k], v), k
  config = pyconfig.from_model_dir(str(tmp_path / "m"), per_device_batch_size=2, max_target_length=40, pagedattn_num_pages=9, pagedattn_tokens_per_page=8)
  assert config.decoder_block == "kifusun" and config.emb_dim == 48 and config.vocab_size == 61 and config.num_decoder_layers == 2
  assert config.embedding_scale == 2.5 and config.normalization_layer_epsilon == 1e-6 and config.attention == "paged"
  plan = kifusun.model_plan(config, loaded)
  l0, l1 = plan["layers"]
  assert (l0["value_mix"], l1["value_mix"]) == (1, 0) and l1["ff"] == 0 and l1["w_gate_up"] is None
  assert torch.equal(l0["w_gate_up"][0::2], tensors["l0.mlp.gate"]) and torch.equal(l0["w_gate_up"][1::2], tensors["l0.mlp.up"])
  assert l0["wqkv"].shape == (4 * 24 + 2 * 24 + 2 * 16, 48) and l0["dist_bias"].shape == (7, 4)
  assert torch.equal(l0["dist_bias"][6], tensors["l0.mix.rel"].float()[ref.distance_bucket(6, 10, 128.0)])


def test_unknown_architecture_and_bad_layers_are_refused():
  cfg = _model([kifusun.attention_layer(4, 2, 8, 8, 4)])
  with pytest.raises(ValueError, match="architecture"):
    pyconfig.from_model_dict(dict(cfg, architecture="Other"))
  bad = _model([kifusun.attention_layer(3, 2, 8, 8, 4)])
  with pytest.raises(ValueError, match="multiple of kv_heads"):
    pyconfig.from_model_dict(bad)
  bad = _model([dict(kifusun.attention_layer(4, 2, 8, 8, 4), type="recurrent")])
  with pytest.raises(ValueError, match="mixer type"):
    pyconfig.from_model_dict(bad)
  bad = _model([kifusun.attention_layer(4, 2, 8, 8, 4), kifusun.attention_layer(4, 2, 8, 16, 4)])
  with pytest.raises(ValueError, match="value mixing"):
    pyconfig.from_model_dict(bad)
  with pytest.raises(ValueError, match="float32"):
    pyconfig.from_model_dict(cfg, dtype="float16")


def test_llama_configs_do_not_take_layered_keys():
  with pytest.raises(ValueError, match="layered"):
    pyconfig.initialize(None, layer_specs=[{"type": "attention"}])


class _Cfg:
  pagedattn_num_pages, pagedattn_tokens_per_page, max_target_length, per_device_batch_size, pagedattn_max_pages_per_group = 8, 4, 24, 3, 6


def test_extend_pages_grows_keeps_and_reuses():
  pm = page_manager.PageManager(_Cfg)
  ps = pm.get_initial_page_state()
  ps = pm.extend_pages(ps, 0, 3)
  assert ps.page_map[0, 0] == 1 and ps.num_pages_used[0] == 1 and ps.sequence_lengths[0] == 3 and ps.has_active_page[0]
  ps = pm.extend_pages(ps, 1, 5)
  assert ps.page_map[1, :2].tolist() == [2, 3]
  ps = pm.extend_pages(ps, 0, 4)  # still inside its page
  assert ps.num_pages_used[0] == 1 and ps.sequence_lengths[0] == 4 and ps.active_page_position[0] == 0
  ps = pm.extend_pages(ps, 0, 9)  # two more pages, the first one kept
  assert ps.page_map[0, :3].tolist() == [1, 4, 5] and ps.active_page[0] == 5 and ps.active_page_position[0] == 1
  ps = pm.release_pages(ps, 1)
  ps = pm.extend_pages(ps, 2, 12)  # the freed pages 2, 3 come first, then 6
  assert ps.page_map[2, :3].tolist() == [2, 3, 6]
  full = pm.extend_pages(ps, 1, 8)  # 2 pages wanted, 1 free (7): nothing changes
  assert full.sequence_lengths[1] == 0 and np.array_equal(full.page_status, ps.page_status)
  assert 0 not in ps.page_map[0, :3].tolist() + ps.page_map[2, :3].tolist()  # page 0 is never handed out
  with pytest.raises(ValueError):
    pm.extend_pages(ps, 0, 2)  # shrinking
  with pytest.raises(ValueError):
    pm.extend_pages(ps, 0, 25)  # beyond max_target_length
  # decoding after a portioned prompt: update_decode_pages continues from what extend_pages left
  ps = pm.release_pages(ps, 2)
  ps = pm.update_decode_pages(ps)
  assert ps.sequence_lengths[0] == 10 and ps.num_pages_used[0] == 3
