"""Fubelorn without a GPU: config.json -> layer table of the layered engine, the registry, and self-checks of the plain oracle (tap
order, mask edges, pooled blocks, frequency scaling, the running maximum, hyper-connections) that the GPU tests lean on."""
import math

import numpy as np
import pytest
import torch

from tests import fubelorn_oracle as fo
from tests.fubelorn_util import config, left_keep, left_pool, mamba2, oracle_logits, parallel, parallel_2, random_weights, right_delta, right_lstm
from xotorch_b200 import _lib
from xotorch_b200.layered import LAYERED_FAMILIES, fubelorn_globals, fubelorn_layers
from xotorch_b200.models import is_layered, model_summary


def test_config_to_layer_table():
  cfg = config([parallel_2(left_pool(heads=6, kv_heads=2, dim=8, vdim=12, size=9, pool=4, rot_dims=4, base=50.0, scaling=(4.0, 1.0, 8.0, 32), scale=0.3),
                           right_lstm(3, 8, 6, cap=7.0), ls=0.6, rs=0.5, ff=40),
                parallel(left_keep(heads=4, kv_heads=4, dim=8, vdim=8, size=11, keep=3), right_delta(4, 2, 8, 6, 3), ls=1.2, rs=0.5, ff=0),
                mamba2(heads=4, vdim=6, state=8, groups=2, norm_groups=3, conv=5, ff=24)], width=48, vocab=80, streams=4, taps=3, mult=0.7)
  a, b, c = fubelorn_layers(cfg, {})
  assert (a.mixer, a.heads, a.kv_heads, a.dim, a.vdim, a.window, a.pool, a.keep_first, a.out_gate, a.qk_norm) == (_lib.LM_MIX_ATTENTION, 6, 2, 8, 12, 9, 4, 0, 1, 0)
  assert (a.rot_dims, a.rot_layout, a.rot_base, a.rot_scale_factor, a.rot_scale_low, a.rot_scale_high, a.rot_scale_original) == (4, _lib.LM_ROT_HALF, 50.0, 4.0, 1.0, 8.0, 32.0)
  assert (a.par_on, a.par_mixer, a.par_heads, a.par_dim, a.par_vdim, a.par_gate_cap) == (1, _lib.LM_MIX_MATRIX_LSTM, 3, 8, 6, 7.0)
  assert abs(a.scale - 0.3) < 1e-12 and (a.mix_scale, a.par_scale, a.ff, a.ff_kind) == (0.6, 0.5, 40, _lib.LM_FF_GELU)
  assert (b.window, b.keep_first, b.pool, b.rot_dims, b.qk_norm, b.out_gate, b.ff) == (11, 3, 0, 0, _lib.LM_QKNORM_HEAD_PLAIN, 0, 0)
  assert (b.par_mixer, b.par_heads, b.par_kv_heads, b.par_dim, b.par_vdim, b.par_conv_taps) == (_lib.LM_MIX_GATED_DELTA, 4, 2, 8, 6, 3)
  assert (c.mixer, c.heads, c.kv_heads, c.dim, c.vdim, c.conv_taps, c.out_norm_groups, c.par_on, c.ff) == (_lib.LM_MIX_MAMBA2, 4, 2, 8, 6, 5, 3, 0, 24)
  g = fubelorn_globals(cfg)
  assert (g["block"], g["streams"], g["canon_taps"], g["residual_mult"], g["embed_norm"]) == (_lib.LM_BLOCK_PRE_SCALAR, 4, 3, 0.7, 1)
  assert is_layered(cfg) and model_summary(cfg)["n_layers"] == 3 and model_summary(cfg)["engine"] == "layered" and "Fubelorn" in LAYERED_FAMILIES
  g = fubelorn_globals(config([mamba2()], streams=None, taps=None))
  assert (g["streams"], g["canon_taps"]) == (0, 0)
  cfg["layers"][2]["type"] = "something_else"
  with pytest.raises(ValueError, match="something_else"):
    fubelorn_layers(cfg, {})
  cfg["layers"][2]["type"] = "mamba2"
  cfg["layers"][0]["mlp"]["kind"] = "sparse"
  with pytest.raises(ValueError, match="sparse"):
    fubelorn_layers(cfg, {})


def test_oracle_convolution_weighs_the_current_token_last():
  x = torch.arange(1.0, 6.0, dtype=torch.float64).reshape(5, 1)
  y = fo.causal_conv(x, torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64))
  assert y.reshape(-1).tolist() == [1.0, 12.0, 123.0, 234.0, 345.0]
  y = fo.causal_conv(x, torch.tensor([[2.0]], dtype=torch.float64), torch.tensor([0.5], dtype=torch.float64))
  assert y.reshape(-1).tolist() == [2.5, 4.5, 6.5, 8.5, 10.5]


def test_oracle_kept_first_tokens_and_window_edges():
  T, size, keep = 12, 4, 2
  i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
  vis = (j <= i) & ((i - j < size) | (j < keep))
  assert vis[11].nonzero().reshape(-1).tolist() == [0, 1, 8, 9, 10, 11] and vis[3].nonzero().reshape(-1).tolist() == [0, 1, 2, 3]
  # the oracle's own mask, read back through identity values
  m = left_keep(heads=1, kv_heads=1, dim=2, vdim=T, size=size, keep=keep, scale=1.0)
  h = torch.eye(T, dtype=torch.float64)
  W = {"q": torch.zeros(2, T, dtype=torch.float64), "k": torch.zeros(2, T, dtype=torch.float64), "v": torch.eye(T, dtype=torch.float64), "o": torch.eye(T, dtype=torch.float64)}
  out = fo.attention_keep_first(h, W, m, 1e-6)
  assert torch.allclose(out[11], vis[11].double() / 6) and torch.allclose(out[5], vis[5].double() / vis[5].sum())


def test_oracle_pooled_blocks_are_seen_once_they_lie_wholly_before_the_window():
  T, size, P = 14, 4, 3
  m = left_pool(heads=1, kv_heads=1, dim=2, vdim=T, size=size, pool=P, rot_dims=0, scaling=None, scale=1.0)
  m.pop("rot")
  h = torch.eye(T, dtype=torch.float64)
  W = {"q": torch.zeros(2, T, dtype=torch.float64), "k": torch.zeros(2, T, dtype=torch.float64), "v": torch.eye(T, dtype=torch.float64), "o": torch.eye(T, dtype=torch.float64),
       "g": torch.zeros(1, T, dtype=torch.float64)}
  out = fo.attention_pooled(h, W, m, 1e-6) * 2           # the gate is sigmoid(0)
  # row 13: tokens 10..13; blocks ending at or before 9: blocks 0, 1, 2 (tokens 0..8); token 9 is seen by nobody.  7 keys share the weight.
  want = torch.zeros(T, dtype=torch.float64)
  want[10:14] = 1 / 7
  want[0:9] = 1 / 7 / 3
  assert torch.allclose(out[13], want)
  # row 6: tokens 3..6; block 0 ends at 2 <= 6 - 4: seen
  want = torch.zeros(T, dtype=torch.float64)
  want[3:7] = 1 / 5
  want[0:3] = 1 / 5 / 3
  assert torch.allclose(out[6], want)
  # row 5: tokens 2..5; block 0 ends at 2 > 5 - 4: not yet
  assert torch.allclose(out[5][:2], torch.zeros(2, dtype=torch.float64)) and torch.allclose(out[5][2:6], torch.full((4,), 0.25, dtype=torch.float64))


def test_oracle_frequency_scaling_bands():
  rot = {"base": 10000.0, "dims": 16, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}
  f0 = [10000.0 ** (-2.0 * i / 16) for i in range(8)]
  f = fo.rotary_frequencies(rot).tolist()
  for a, b in zip(f0, f):
    wl = 2 * math.pi / a
    if wl < 16:
      assert b == a
    elif wl > 64:
      assert abs(b - a / 8) < 1e-15
    else:
      s = (64 / wl - 1) / 3
      assert abs(b - ((1 - s) * a / 8 + s * a)) < 1e-15 and a / 8 < b < a
  assert f[0] == 1.0 and abs(f[-1] - f0[-1] / 8) < 1e-15 and any(a / 8 < b < a for a, b in zip(f0, f)), "all three bands are met"


def test_oracle_rotation_depends_on_the_distance_only():
  f = fo.rotary_frequencies({"base": 10.0, "dims": 4})
  g = torch.Generator().manual_seed(1)
  q, k = torch.randn(1, 1, 6, dtype=torch.float64, generator=g), torch.randn(1, 1, 6, dtype=torch.float64, generator=g)
  dot = lambda pq, pk: float((fo.rotate_half_layout(q, torch.tensor([pq]), f, 4) * fo.rotate_half_layout(k, torch.tensor([pk]), f, 4)).sum())
  assert abs(dot(9, 4) - dot(105, 100)) < 1e-9 and abs(dot(9, 4) - dot(9, 5)) > 1e-3
  assert torch.equal(fo.rotate_half_layout(q, torch.tensor([7]), f, 4)[..., 4:], q[..., 4:]), "entries beyond the rotated ones pass"


def test_oracle_matrix_lstm_by_hand():
  """one head, sizes 1: with q = k = v = 1 the state is a number.  i = 0, f = logsigmoid(0) = -ln 2 at every token (cap large)."""
  m = right_lstm(1, 1, 1, cap=50.0)
  h = torch.ones(3, 1, dtype=torch.float64)
  one, zero = torch.ones(1, 1, dtype=torch.float64), torch.zeros(1, 1, dtype=torch.float64)
  W = {"q": one, "k": one, "v": one, "i": zero, "f": zero, "i.b": torch.zeros(1, dtype=torch.float64), "f.b": torch.zeros(1, dtype=torch.float64),
       "g": zero, "norm": torch.ones(1, dtype=torch.float64), "o": one}
  # m_t = max(-ln2 + m, 0) = 0; S_t = S/2 + 1 -> 1, 1.5, 1.75; n the same; o = S / (max(n, 1) + 1e-6) ~ 1 -> rms norm -> 1 -> gate 1/2
  out = fo.matrix_lstm(h, W, m, 0.0)
  assert torch.allclose(out.reshape(-1), torch.full((3,), 0.5, dtype=torch.float64), atol=1e-6)
  # a large input gate lifts the maximum: i = 5 -> m_1 = 5, S_1 = e^0 k v = 1, floor e^-5 is below n = 1
  W["i.b"] = torch.tensor([5.0], dtype=torch.float64)
  out = fo.matrix_lstm(h, W, m, 0.0)
  assert torch.allclose(out.reshape(-1), torch.full((3,), 0.5, dtype=torch.float64), atol=1e-6)


def test_oracle_hyper_connections_with_identity_coefficients_are_the_plain_residual():
  cfg1 = config([parallel(), mamba2()], streams=1)
  cfg0 = config([parallel(), mamba2()], streams=None)
  W = random_weights(cfg1, 3)
  for k in list(W):
    if ".hc" in k:
      W[k] = torch.ones_like(W[k])
  toks = np.arange(17) % cfg1["vocab"]
  a = oracle_logits(cfg1, W, toks)[0]
  b = oracle_logits(cfg0, {k: v for k, v in W.items() if ".hc" not in k}, toks)[0]
  assert np.allclose(a, b, atol=1e-10)


def test_oracle_is_causal():
  cfg = config([parallel_2(), parallel(), mamba2()])
  W = random_weights(cfg, 5)
  toks = np.arange(30) % cfg["vocab"]
  a = oracle_logits(cfg, W, toks)[0]
  b = oracle_logits(cfg, W, toks[:19])[0]
  assert np.allclose(a[:19], b, atol=1e-9)
