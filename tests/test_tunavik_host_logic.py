"""Host-side logic of the Tunavik family (no GPU): config.json -> layer table, the registry, and self-checks of the plain oracle
that the GPU tests compare the engine with."""
import math

import numpy as np
import pytest
import torch

from tests import tunavik_oracle as to
from tests.tunavik_util import attention, config, moe
from xotorch_b200 import _lib
from xotorch_b200.layered import LAYERED_FAMILIES, tunavik_globals, tunavik_layers
from xotorch_b200.models import is_layered, model_summary


def test_config_becomes_a_layer_table():
  cfg = config([attention(heads=6, kv_heads=3, dim=10, vdim=4, bias_max=77, temp=(0.25, 9), mlp=moe(5, 3, 14, 22)),
                attention(heads=6, kv_heads=3, dim=10, vdim=4, temp=None, kv_from=0, mlp=None),
                attention(heads=2, kv_heads=2, dim=8, vdim=8, mlp=moe(4, 1, 8, None))], width=40, vocab=91, logit_scale=None, softcap=None)
  shapes = to.tensor_shapes(cfg, buckets=[12, 6, 2])
  a, b, c = tunavik_layers(cfg, shapes)
  assert (a.mixer, a.heads, a.kv_heads, a.dim, a.vdim, a.kv_from) == (_lib.LM_MIX_ATTENTION, 6, 3, 10, 4, -1)
  assert (a.qk_norm, a.proj_bias, a.out_bias, a.sink) == (_lib.LM_QKNORM_ROW, 1, 1, 1)
  assert (a.rel_buckets, a.rel_max, a.q_temp_coef, a.q_temp_every) == (12, 77.0, 0.25, 9)
  assert (a.ff_kind, a.experts, a.top, a.expert_ff, a.shared_ff) == (_lib.LM_FF_MOE, 5, 3, 14, 22)
  assert (a.expert_act, a.router_kind, a.router_bias) == (_lib.LM_EXPERT_RELU2, _lib.LM_ROUTER_TOPK_SOFTMAX, 1)
  assert (b.kv_from, b.rel_buckets, b.q_temp_coef, b.experts) == (0, 6, 0.0, 0)     # no temperature, no feed-forward
  assert (c.rel_buckets, c.top, c.shared_ff) == (2, 1, 0)
  g = tunavik_globals(cfg)
  assert g["block"] == _lib.LM_BLOCK_POST_RMS and g["pos_sinusoid"] == 1 and g["embed_norm"] == 1
  assert g["logit_scale"] == 1.0 and g["logit_softcap"] == 0.0                      # absent keys: nothing is scaled or capped
  g = tunavik_globals(config([attention()], logit_scale=0.3, softcap=11.0))
  assert (g["logit_scale"], g["logit_softcap"]) == (0.3, 11.0)


def test_registry_knows_the_family():
  cfg = config([attention(mlp=moe())], width=24, vocab=33)
  assert "Tunavik" in LAYERED_FAMILIES and is_layered(cfg)
  s = model_summary(cfg)
  assert (s["n_layers"], s["vocab"], s["width"], s["engine"]) == (1, 33, 24, "layered")


def test_unknown_layer_kinds_are_refused():
  cfg = config([attention()])
  shapes = to.tensor_shapes(cfg)
  bad = config([attention()])
  bad["layers"][0]["type"] = "delta"
  with pytest.raises(ValueError, match="delta"):
    tunavik_layers(bad, shapes)
  bad = config([attention(mlp={"kind": "dense", "ff": 8})])
  with pytest.raises(ValueError, match="dense"):
    tunavik_layers(bad, shapes)
  with pytest.raises(ValueError, match="rel"):
    tunavik_layers(cfg, {})                           # the number of buckets comes from the table's shape


# ---- the oracle's own mechanisms ---------------------------------------------------------------------------------------------
def test_oracle_distance_buckets():
  for B, far in ((16, 200.0), (8, 20.0), (2, 5.0), (6, 1000.0)):
    b = [to.distance_bucket(n, B, far) for n in range(int(far) + 50)]
    assert b[:B // 2] == list(range(B // 2))                      # near distances: one bucket each
    assert all(y - x in (0, 1) or x < B // 2 for x, y in zip(b, b[1:])) and b == sorted(b)
    assert b[int(far)] == B - 1 and max(b) == B - 1               # the last bucket is reached at `far` at the latest
    assert b[B // 2] == B // 2
  # 8 buckets up to distance 20: the logarithmic half has its edges at 4 * 5^(k/4) = 4, 5.98, 8.94, 13.4, 20
  assert [to.distance_bucket(n, 8, 20.0) for n in (4, 5, 6, 8, 9, 13, 14, 19, 20)] == [4, 4, 5, 5, 6, 6, 7, 7, 7]


def test_oracle_query_temperature_steps():
  t = to.query_temperature(40, 2.0, 8, torch.float64)
  assert torch.all(t[:7] == 1.0) and t[7] == 1.0 + 2.0 * math.log(2) and t[14] == t[7] and t[15] == 1.0 + 2.0 * math.log(3)


def test_oracle_sink_takes_weight_and_gives_no_value():
  cfg = config([attention(heads=2, kv_heads=1, dim=4, vdim=4, temp=None)], width=16)
  W = to.random_weights(cfg, 1)
  Wm = to.sub({k: v.double() for k, v in W.items()}, "l0.mix.")
  m = cfg["layers"][0]["mixer"]
  h = torch.randn(5, 16, dtype=torch.float64)
  Wm["o"], Wm["o.b"] = torch.eye(16, 8, dtype=torch.float64), torch.zeros(16, dtype=torch.float64)
  Wm["sink"] = torch.full((2,), -60.0, dtype=torch.float64)
  plain = to.attention(h, Wm, m, 1e-5)
  _, v = to.attention_keys_values(h, Wm, m, 1e-5)
  assert torch.allclose(plain[0, :4], v[0, 0])                    # first token, no sink to speak of: all weight on itself
  Wm["sink"] = torch.full((2,), 60.0, dtype=torch.float64)
  assert to.attention(h, Wm, m, 1e-5).abs().max() < 1e-12         # a huge sink takes everything: nothing is read


def test_oracle_routing():
  r = {"experts": 5, "top": 3}
  W = {"router": torch.eye(5, 5, dtype=torch.float64), "router.b": torch.tensor([0.0, 0.0, 10.0, 0.0, 0.0], dtype=torch.float64)}
  h = torch.tensor([[3.0, 1.0, -5.0, 2.0, 0.0]], dtype=torch.float64)
  ids, w = to.route(h, W, r)
  assert ids.tolist() == [[2, 0, 3]]                              # the bias decides: logits 3, 1, 5, 2, 0
  assert torch.allclose(w, torch.softmax(torch.tensor([[5.0, 3.0, 2.0]], dtype=torch.float64), -1)) and abs(float(w.sum()) - 1) < 1e-12


def test_oracle_positions_and_norm():
  pv = to.position_vectors(7, 6, torch.float64)
  assert torch.allclose(pv[0], torch.tensor([0.0, 1.0] * 3, dtype=torch.float64))
  assert abs(float(pv[3, 2]) - math.sin(3 * 10000.0 ** (-2 / 6))) < 1e-12 and abs(float(pv[3, 5]) - math.cos(3 * 10000.0 ** (-4 / 6))) < 1e-12
  x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
  assert torch.allclose(to.norm_around_zero(x, torch.tensor([0.0, 1.0], dtype=torch.float64), 0.0), torch.tensor([[3.0, 8.0]], dtype=torch.float64) / math.sqrt(12.5))


def test_oracle_portions_do_not_exist_but_prefixes_agree():
  """the oracle has no cache: the logits of a prefix are the first rows of the longer sequence's logits (causality)"""
  cfg = config([attention(mlp=moe()), attention(kv_from=0, mlp=None)])
  W = to.random_weights(cfg, 3)
  toks = np.random.default_rng(0).integers(0, cfg["vocab"], 30)
  full, _ = to.forward(cfg, W, toks)
  part, _ = to.forward(cfg, W, toks[:11])
  assert torch.allclose(full[:11], part, atol=1e-10)
