"""The Fubelorn family on the layered engine (libxotb200_lm.so) against the plain oracle (tests/fubelorn_oracle.py) on small random
models (-m gpu).  The float32 engine is held to the oracle in float64 tightly, the bfloat16 engine loosely; tests ask for the
logits of EVERY row unless they say otherwise, so a wrong key, window edge, pooled block, lost state or stream shows at any place."""
import json
import struct

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from tests.fubelorn_util import (config, left_keep, left_pool, mamba2, oracle_logits, parallel, parallel_2, random_weights, right_delta, right_lstm)
from tests.layered_util import TOL, bf16_bits, make_engine, rand_tokens, row_err, run_cut

DTYPES = ["float32", "bfloat16"]

MIXED = [parallel_2(left_pool(heads=4, kv_heads=2, dim=8, vdim=12, size=9, pool=4, rot_dims=8), right_lstm(3, 8, 6)),
         parallel(left_keep(heads=4, kv_heads=4, dim=8, vdim=8, size=11, keep=3), right_delta(4, 2, 8, 6, 3)),
         mamba2(heads=4, vdim=6, state=8, groups=2, norm_groups=2, conv=3),
         parallel(left_keep(heads=2, kv_heads=1, dim=12, vdim=10, size=6, keep=2), right_delta(2, 2, 6, 10, 2), ff=0),
         parallel_2(left_pool(heads=3, kv_heads=3, dim=12, vdim=6, size=7, pool=3, rot_dims=6, scaling=None), right_lstm(2, 6, 10, cap=8.0))]


def check(native, cfg, W, tokens, cuts, dtype, slot=0, tol=None):
  ref, _ = oracle_logits(cfg, W, tokens)
  got = run_cut(native, slot, tokens, cuts)
  e = row_err(got, ref)
  assert e < (tol or TOL[dtype]), f"{dtype}: rows differ from the oracle, worst relative error {e:.3e}"
  return got


# ---- each mechanism alone ------------------------------------------------------------------------------------------------
SINGLE = {
  "kept_first_attention_and_delta": ([parallel()], {}),
  "kept_first_one_kv_head": ([parallel(left_keep(heads=6, kv_heads=1, dim=8, vdim=8))], {}),
  "kept_first_none_kept": ([parallel(left_keep(keep=0))], {}),
  "kept_first_more_than_window": ([parallel(left_keep(size=4, keep=7))], {}),
  "window_of_one": ([parallel(left_keep(size=1, keep=1))], {}),
  "window_beyond_the_prompt": ([parallel(left_keep(size=500, keep=2))], {}),
  "attention_odd_sizes": ([parallel(left_keep(heads=3, kv_heads=3, dim=5, vdim=3), right_delta(3, 1, 5, 7, 4))], {"width": 36}),
  "attention_wide_values": ([parallel(left_keep(heads=2, kv_heads=1, dim=40, vdim=72))], {}),
  "attention_very_wide_values": ([parallel_2(left_pool(heads=2, kv_heads=2, dim=24, vdim=328, rot_dims=12))], {}),
  "delta_one_tap": ([parallel(right=right_delta(2, 2, 8, 8, 1))], {}),
  "delta_seven_taps": ([parallel(right=right_delta(4, 1, 4, 12, 7))], {}),
  "pooled_attention_and_lstm": ([parallel_2()], {}),
  "pooled_blocks_of_one": ([parallel_2(left_pool(size=5, pool=1))], {}),
  "pooled_blocks_longer_than_window": ([parallel_2(left_pool(size=3, pool=7))], {}),
  "pooled_window_of_one": ([parallel_2(left_pool(size=1, pool=2))], {}),
  "rotation_of_half_the_head": ([parallel_2(left_pool(dim=16, rot_dims=8))], {}),
  "rotation_without_scaling": ([parallel_2(left_pool(scaling=None))], {}),
  "rotation_scaling_band": ([parallel_2(left_pool(dim=32, base=10000.0, scaling=(8.0, 1.0, 4.0, 64)))], {}),
  "lstm_one_head": ([parallel_2(right=right_lstm(1, 16, 4))], {}),
  "lstm_small_cap": ([parallel_2(right=right_lstm(3, 8, 6, cap=2.0))], {}),
  "lstm_odd_sizes": ([parallel_2(left_pool(heads=3, kv_heads=3, dim=6, vdim=5, rot_dims=4), right_lstm(5, 7, 3))], {"width": 36}),
  "state_space": ([mamba2()], {}),
  "state_space_one_group": ([mamba2(heads=6, vdim=4, state=16, groups=1, norm_groups=1, conv=4)], {}),
  "state_space_group_per_head": ([mamba2(heads=3, vdim=8, state=5, groups=3, norm_groups=4, conv=2)], {}),
  "state_space_one_tap": ([mamba2(conv=1)], {}),
  "no_feed_forward_anywhere": ([parallel(ff=0), mamba2(ff=0), parallel_2(ff=0)], {}),
  "one_stream": ([parallel(), parallel_2()], {"streams": 1}),
  "plain_residual_stream": ([parallel(), mamba2()], {"streams": None}),
  "eight_streams": ([parallel_2(), mamba2()], {"streams": 8}),
  "no_input_convolution": ([parallel(), parallel_2()], {"taps": None}),
  "input_convolution_of_one_tap": ([parallel(), mamba2()], {"taps": 1}),
  "input_convolution_of_six_taps": ([parallel_2(), mamba2()], {"taps": 6}),
  "unit_multiplier_and_scales": ([parallel(ls=1.0, rs=1.0)], {"mult": 1.0}),
  "width_not_a_multiple_of_four": ([parallel(), parallel_2(), mamba2()], {"width": 30, "streams": 2}),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_one_mechanism_models(name, dtype):
  layers, kw = SINGLE[name]
  cfg = config(layers, **kw)
  W = random_weights(cfg, 11)
  n = make_engine(cfg, W, dtype)
  toks = rand_tokens(cfg["vocab"], 41, 3)
  n.set_trace(True)
  ref, trail = oracle_logits(cfg, W, toks)
  got, _ = n.step([0], [toks], want=list(range(len(toks))))
  x = n.read_trace(len(toks))
  for i, t in enumerate(trail):
    assert np.abs(x[i] - t).max() / np.abs(t).max() < (1e-5 if dtype == "float32" else 0.03), f"stream after layer {i} differs"
  assert row_err(got, ref) < TOL[dtype]
  n.set_trace(False)
  cut = run_cut(n, 1, toks, [7, 5, 1])               # short portions and single rows: cache and states carried between steps
  assert row_err(cut, ref) < TOL[dtype]
  n.close()


# ---- prefill / decoding / portions -----------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cuts", [[1], [2], [3], [17, 1], [5, 2, 9, 1], [64]])
def test_portions_equal_the_whole_prompt(cuts, dtype):
  cfg = config(MIXED)
  W = random_weights(cfg, 2)
  n = make_engine(cfg, W, dtype, page_size=4)
  toks = rand_tokens(cfg["vocab"], 37, 8)
  got = check(n, cfg, W, toks, cuts, dtype)
  n.clear_request(0)
  whole = run_cut(n, 0, toks, [len(toks)])
  assert row_err(got, whole.astype(np.float64)) < (2e-5 if dtype == "float32" else 0.05), "cutting the prompt changes rounding only"
  n.close()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype):
  """300 tokens, all but six decoded one by one: windows pass over decoded tokens, blocks are completed and pooled by single rows,
  the keys of a decode step are cut into runs, the recurrent states are carried 294 times"""
  cfg = config([parallel_2(left_pool(size=40, pool=6)), parallel(left_keep(size=50, keep=4)), mamba2()], width=32)
  W = random_weights(cfg, 21)
  n = make_engine(cfg, W, dtype, max_tokens=400, page_size=16)
  check(n, cfg, W, rand_tokens(cfg["vocab"], 300, 4), [6, 1], dtype)
  n.close()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_prompt_then_decoding_in_a_batch_of_unequal_requests(dtype):
  """a mid-sized model (blocks of 10 that do not divide the 64-token pages, windows of 70 and 90, 5 kept tokens, partial rotation, grouped
  state-space layer first) on 650 / 300 / 41 tokens: each prompt whole in one batch, then 30 tokens decoded together, the short request
  ending early — far keys, many pooled blocks, key runs over several CTAs, states carried over hundreds of tokens"""
  cfg = config([mamba2(heads=6, vdim=16, state=24, groups=2, norm_groups=3, conv=4, ff=96),
                parallel_2(left_pool(heads=6, kv_heads=2, dim=32, vdim=40, size=70, pool=10, rot_dims=16, base=5000.0, scaling=(4.0, 1.0, 4.0, 256)),
                           right_lstm(3, 24, 32, cap=10.0), ff=96),
                parallel(left_keep(heads=3, kv_heads=3, dim=24, vdim=24, size=90, keep=5), right_delta(6, 3, 16, 24, 4), ff=0),
                parallel_2(left_pool(heads=4, kv_heads=1, dim=16, vdim=56, size=33, pool=7, rot_dims=16, scaling=None), right_lstm(2, 32, 16), ff=64)],
               width=120, vocab=300, streams=4, taps=4, mult=0.6)
  W = random_weights(cfg, 77)
  lens, extra = [650, 300, 41], 30
  seqs = [rand_tokens(cfg["vocab"], L + extra, 90 + i) for i, L in enumerate(lens)]
  refs = [oracle_logits(cfg, W, s)[0] for s in seqs]
  n = make_engine(cfg, W, dtype, max_tokens=1200, max_requests=3, page_size=64)
  want = [0, 1, 64, 500, 649, 650 + 0, 650 + 128, 650 + 299, 950 + 40]
  lg, _ = n.step([0, 1, 2], [s[:L] for s, L in zip(seqs, lens)], want=want)
  ref = np.stack([refs[0][0], refs[0][1], refs[0][64], refs[0][500], refs[0][649], refs[1][0], refs[1][128], refs[1][299], refs[2][40]])
  assert rows_agree(lg, ref, dtype), "prompts"
  live, dec = [0, 1, 2], {0: [], 1: [], 2: []}
  for t in range(extra):
    if t == 12:
      live.remove(2)
      n.clear_request(2)
    lg, _ = n.step(live, [seqs[i][lens[i] + t:lens[i] + t + 1] for i in live])
    for k, i in enumerate(live):
      dec[i].append(lg[k])
  for i in range(3):
    got = np.stack(dec[i])
    assert rows_agree(got, refs[i][lens[i]:lens[i] + len(got)], dtype), f"decoded tokens of request {i}"
  n.close()


def test_first_tokens_of_a_sequence():
  cfg = config(MIXED)
  W = random_weights(cfg, 9)
  n = make_engine(cfg, W, "float32")
  for length in (1, 2, 3, 5):
    n.clear_request(0)
    check(n, cfg, W, rand_tokens(cfg["vocab"], length, length), [1], "float32")
    n.clear_request(0)
    check(n, cfg, W, rand_tokens(cfg["vocab"], length, length), [length], "float32")
  n.close()


# ---- batches ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_requests_in_one_batch_equal_each_alone(dtype):
  cfg = config(MIXED)
  W = random_weights(cfg, 4)
  n = make_engine(cfg, W, dtype, max_tokens=256, max_requests=5, page_size=4)
  lens = [1, 13, 30, 2, 8]
  seqs = [rand_tokens(cfg["vocab"], L + 6, 50 + i) for i, L in enumerate(lens)]
  refs = [oracle_logits(cfg, W, s)[0] for s in seqs]
  slots = [3, 0, 4, 1, 2]
  lg, _ = n.step(slots, [s[:L] for s, L in zip(seqs, lens)], want=list(range(sum(lens))))
  at = 0
  for i, L in enumerate(lens):
    assert row_err(lg[at:at + L], refs[i][:L]) < TOL[dtype], f"prompt of request {i}"
    at += L
  live = list(range(len(lens)))
  for t in range(6):
    if t == 2:
      live.remove(0)
      n.clear_request(slots[0])
    if t == 4:
      live.remove(3)
      n.clear_request(slots[3])
    lg, am = n.step([slots[i] for i in live], [seqs[i][lens[i] + t:lens[i] + t + 1] for i in live])
    for k, i in enumerate(live):
      assert row_err(lg[k:k + 1], refs[i][lens[i] + t:lens[i] + t + 1]) < TOL[dtype], f"request {i}, decoded token {t}"
      assert am[k] == int(np.argmax(lg[k]))
  n.close()


def test_mixed_batch_of_portions_and_decoded_rows():
  cfg = config(MIXED)
  W = random_weights(cfg, 6)
  n = make_engine(cfg, W, "float32", page_size=4)
  a, b = rand_tokens(cfg["vocab"], 20, 1), rand_tokens(cfg["vocab"], 26, 2)
  ra, rb = oracle_logits(cfg, W, a)[0], oracle_logits(cfg, W, b)[0]
  n.step([0], [a[:15]])
  lg, _ = n.step([0, 1], [a[15:16], b[:11]], want=list(range(12)))
  assert row_err(lg[:1], ra[15:16]) < TOL["float32"] and row_err(lg[1:], rb[:11]) < TOL["float32"]
  lg, _ = n.step([1, 0], [b[11:26], a[16:17]], want=list(range(16)))
  assert row_err(lg[:15], rb[11:26]) < TOL["float32"] and row_err(lg[15:], ra[16:17]) < TOL["float32"]
  n.close()


# ---- pages, slots and states that are given back and used again ----------------------------------------------------------------
def test_freed_pages_slots_and_states_are_clean_for_the_next_request():
  cfg = config(MIXED)
  W = random_weights(cfg, 13)
  n = make_engine(cfg, W, "float32", max_tokens=64, max_requests=2, page_size=4)
  total = n.cache_stats()["pages_total"]
  a, b, c = (rand_tokens(cfg["vocab"], L, s) for L, s in ((29, 1), (18, 2), (31, 3)))
  check(n, cfg, W, a, [9, 1], "float32", slot=0)
  check(n, cfg, W, b, [18], "float32", slot=1)
  assert n.cache_stats()["pages_free"] == total - 8 - 5
  n.clear_request(0)                                  # a's pages go back, its states (matrices, maxima, filter inputs) are zeroed ...
  assert n.cache_stats()["pages_free"] == total - 5 and n.request_len(0) == 0
  check(n, cfg, W, c, [5, 3, 1], "float32", slot=0)   # ... and c starts clean on them, next to the live b
  lg, _ = n.step([1], [a[:3]], want=[0, 1, 2])        # b goes on undisturbed
  ref = oracle_logits(cfg, W, np.concatenate([b, a[:3]]))[0]
  assert row_err(lg, ref[18:]) < TOL["float32"]
  n.clear_request(0)
  n.clear_request(1)
  assert n.cache_stats()["pages_free"] == total
  with pytest.raises(Exception, match="cache"):
    n.step([0], [rand_tokens(cfg["vocab"], 200, 1)])
  assert n.cache_stats()["pages_free"] == total and n.request_len(0) == 0
  n.close()


# ---- keys made to stand out: far away, at page borders, at the edges of windows, kept tokens and pooled blocks ---------------------
def plant(cfg, W, dims):
  """The last two tokens of the vocabulary get embeddings made for each other: the key of the first and every query of the second
  point along one sign vector on the head entries `dims` (the first layer's projections are inverted for it; the norms in front
  of them keep directions), so that this pair's score stands out from all others."""
  m, V = cfg["layers"][0]["mixer"]["left"], cfg["vocab"]
  u = torch.zeros(m["dim"], dtype=torch.float64)
  u[dims] = torch.tensor([1.0, -1.0] * (len(dims) // 2), dtype=torch.float64)
  k_dir = torch.linalg.pinv(W["l0.mix.left.k"].double()) @ u.repeat(m["kv_heads"])
  q_dir = torch.linalg.pinv(W["l0.mix.left.q"].double()) @ u.repeat(m["heads"])
  W["embed"][V - 2] = (k_dir / k_dir.norm() * W["embed"].shape[1] ** 0.5).to(torch.bfloat16).float()
  W["embed"][V - 1] = (q_dir / q_dir.norm() * W["embed"].shape[1] ** 0.5).to(torch.bfloat16).float()
  return V - 2, V - 1


def planted_case(layer, dims, pos, n_tok, dtype, decode, page, must_matter, seed=17):
  V = 40
  layer["mixer"]["right_scale"] = 0.0                   # the attention branch alone carries the planted pair
  cfg = config([layer], vocab=V, width=64, streams=2, taps=2)
  W = random_weights(cfg, seed, canon_gain=0.05)
  key_tok, query_tok = plant(cfg, W, dims)
  seq = rand_tokens(V - 2, n_tok, 5)
  seq[-1] = query_tok
  without = oracle_logits(cfg, W, seq)[0]
  seq[np.atleast_1d(pos)] = key_tok
  ref = oracle_logits(cfg, W, seq)[0]
  gain = row_err(ref[-1:], without[-1:])
  if must_matter:
    assert gain > 0.2, f"the planted key does not stand out ({gain})"
  n = make_engine(cfg, W, dtype, max_tokens=512, page_size=page)
  got = run_cut(n, 0, seq, [n_tok - 40, 1] if decode else [n_tok])
  e = row_err(got[-1:], ref[-1:])
  assert e < TOL[dtype], f"key at {pos} of {n_tok} ({'decoded' if decode else 'prompt'}): {e:.3e} (the key moves the row by {gain:.2e})"
  assert row_err(got, ref) < TOL[dtype]
  n.close()
  return gain


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
def test_kept_tokens_window_edges_and_page_borders(decode, dtype):
  """window 64, the first 5 tokens kept, 150 tokens: the last row (position 149) sees 0..4 and 86..149.  One key made to dominate it sits
  on the last kept token, on the first token that is not kept, on the oldest token inside the window, on the newest outside it, and
  on either side of a page border inside the window."""
  n_tok, size, keep = 150, 64, 5
  for name, pos, page, matters in (("first_in", keep - 1, 16, True), ("first_out", keep, 16, False), ("window_in", n_tok - size, 16, True),
                                   ("window_out", n_tok - size - 1, 16, False), ("page_first", 128, 64, True), ("page_last", 127, 64, True),
                                   ("second_token", 1, 8, True)):
    layer = parallel(left_keep(heads=2, kv_heads=1, dim=16, vdim=16, size=size, keep=keep, scale=1.2))
    gain = planted_case(layer, list(range(16)), pos, n_tok, dtype, decode, page, matters)
    if not matters:
      assert gain < 0.05, f"{name}: the oracle itself sees the key ({gain})"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
def test_pooled_blocks_window_edges_and_far_keys(decode, dtype):
  """window 48, blocks of 4, 150 tokens, rotation on the first half of a head (the planted pair lives on the other half, where positions
  do not enter): the last row (149) sees tokens 102..149 and the blocks that end at or before 101, i.e. blocks 0..24 (tokens 0..99);
  tokens 100 and 101 are seen by nobody.  A pooled key is the mean of four, so a whole block is planted: the newest block seen, the
  gap, the oldest token of the window, block 0 far away, a block whose pooled row starts a page, and a token at a page border."""
  n_tok, size, P = 150, 48, 4
  for name, pos, page, matters in (("pool_in", [96, 97, 98, 99], 16, True), ("gap", [100, 101], 16, False), ("window_in", 102, 16, True),
                                   ("far", [0, 1, 2, 3], 16, True), ("pooled_row_starts_a_page", [32, 33, 34, 35], 8, True),
                                   ("pooled_row_ends_a_page", [28, 29, 30, 31], 8, True), ("page_border_token", 128, 64, True)):
    layer = parallel_2(left_pool(heads=2, kv_heads=1, dim=16, vdim=16, size=size, pool=P, rot_dims=8, scale=1.0))
    gain = planted_case(layer, list(range(8, 16)), pos, n_tok, dtype, decode, page, matters)
    if not matters:
      assert gain < 0.05, f"{name}: the oracle itself sees the key ({gain})"


def test_rotation_follows_the_position_in_the_sequence():
  """a strongly rotating layer (small base, whole head turned): a portion that starts at position 13 must turn its queries and keys by
  their places in the sequence, not in the portion"""
  cfg = config([parallel_2(left_pool(heads=2, kv_heads=2, dim=8, vdim=8, size=40, pool=5, base=3.0, scaling=None, scale=1.0))], width=32)
  W = random_weights(cfg, 31)
  toks = rand_tokens(cfg["vocab"], 60, 9)
  n = make_engine(cfg, W, "float32", page_size=8)
  check(n, cfg, W, toks, [13, 20, 1], "float32")
  n.close()


def test_running_maximum_of_the_matrix_lstm_is_carried():
  """input gates far above the forget gates' decay: the running maximum climbs, the floor e^(-m) of the normaliser matters early and
  the normaliser later; prompts, portions and decoding must agree with the oracle"""
  cfg = config([parallel_2(right=right_lstm(2, 8, 8, cap=12.0), ls=0.1, rs=1.5)], width=32)
  W = random_weights(cfg, 37)
  W["l0.mix.right.i.b"] = torch.tensor([6.0, -6.0])
  W["l0.mix.right.f.b"] = torch.tensor([-3.0, 5.0])
  toks = rand_tokens(cfg["vocab"], 70, 2)
  n = make_engine(cfg, W, "float32", page_size=8)
  check(n, cfg, W, toks, [70], "float32", slot=0)
  check(n, cfg, W, toks, [33, 2, 1], "float32", slot=1)
  n.close()


def rows_agree(got, ref, dtype):
  """float32: every row within the tolerance.  bfloat16: the models drawn at random are not chosen for their conditioning, so up to
  5 % of the rows may leave the tolerance (by less than a factor of two) while the median row stays within a third of it."""
  if dtype == "float32":
    return row_err(got, ref) < TOL[dtype]
  e = np.array([row_err(got[i:i + 1], ref[i:i + 1]) for i in range(len(ref))])
  return np.median(e) < TOL[dtype] / 3 and (e > TOL[dtype]).mean() <= 0.05 and e.max() < 2 * TOL[dtype]


# ---- models drawn at random --------------------------------------------------------------------------------------------------------
def draw_model(seed):
  r = np.random.default_rng(seed)
  pick = lambda *xs: xs[int(r.integers(len(xs)))]
  layers = []
  for _ in range(int(r.integers(2, 5))):
    kind = pick("parallel", "parallel_2", "mamba2")
    ff = pick(0, 24, 40)
    if kind == "mamba2":
      G = pick(1, 2, 3)
      H = G * pick(1, 2)
      dv = pick(4, 6, 8)
      ng = pick(1, 2, H)
      layers.append(mamba2(heads=H, vdim=dv, state=pick(4, 8, 12), groups=G, norm_groups=ng if (H * dv) % ng == 0 else 1, conv=pick(1, 2, 4), ff=ff))
      continue
    G = pick(1, 2, 3)
    H, d, dv = G * pick(1, 2, 4), pick(4, 8, 12, 16), pick(4, 8, 10)
    if kind == "parallel":
      rg = pick(1, 2)
      layers.append(parallel(left_keep(H, G, d, dv, size=pick(1, 5, 16, 33), keep=pick(0, 1, 4, 9)),
                             right_delta(rg * pick(1, 2), rg, pick(4, 8), pick(4, 6), pick(1, 3, 4)), ls=pick(0.5, 1.2), rs=pick(0.5, 1.0), ff=ff))
    else:
      layers.append(parallel_2(left_pool(H, G, d, dv, size=pick(2, 7, 20), pool=pick(1, 3, 8), rot_dims=pick(d, d // 2, 2),
                                         scaling=pick(None, (4.0, 1.0, 4.0, 16), (2.0, 0.5, 8.0, 64))),
                               right_lstm(pick(1, 2, 4), pick(4, 8), pick(4, 6), cap=pick(5.0, 15.0)), ls=pick(0.6, 1.0), rs=pick(0.5, 1.1), ff=ff))
  return config(layers, width=pick(32, 40, 48), vocab=64, streams=pick(None, 1, 2, 4), taps=pick(None, 2, 4), mult=pick(0.5, 0.7, 1.0))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed", range(8))
def test_models_drawn_at_random(seed, dtype):
  cfg = draw_model(seed)
  W = random_weights(cfg, 100 + seed)
  n = make_engine(cfg, W, dtype, max_tokens=256, max_requests=3, page_size=8)
  a, b = rand_tokens(cfg["vocab"], 70, seed), rand_tokens(cfg["vocab"], 9, seed + 50)
  ra, rb = oracle_logits(cfg, W, a)[0], oracle_logits(cfg, W, b)[0]
  lg, _ = n.step([2, 0], [a[:45], b[:4]], want=list(range(49)))
  assert rows_agree(lg[:45], ra[:45], dtype) and rows_agree(lg[45:], rb[:4], dtype)
  dec = []
  for t in range(5):
    lg, _ = n.step([0, 2], [b[4 + t:5 + t], a[45 + t:46 + t]])
    dec.append(lg)
  dec = np.stack(dec)
  assert rows_agree(dec[:, 0], rb[4:9], dtype) and rows_agree(dec[:, 1], ra[45:50], dtype), "decoded tokens"
  lg, _ = n.step([2], [a[50:]], want=list(range(20)))
  assert rows_agree(lg, ra[50:], dtype), "late portion"
  n.close()


# ---- kernel variants ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("sizes", [(16, 16, 70, 5, 33, 4), (24, 8, 64, 64, 64, 64), (8, 40, 1, 0, 2, 1), (16, 72, 130, 9, 100, 7)])
def test_tensor_core_prompt_attention_equals_the_plain_kernel(sizes):
  """bfloat16, head sizes that are whole 16-byte pieces: portions of 16 rows or more take the tensor-core streaming-softmax kernel, which
  walks kept first tokens / pooled blocks in front of the window's tokens; it must agree with the warp-per-row kernel and the oracle
  (prompt of 200 rows, then a late portion of 60 that starts inside the sequence)"""
  d, dv, size, keep, size2, P = sizes
  cfg = config([parallel(left_keep(heads=4, kv_heads=2, dim=d, vdim=dv, size=size, keep=keep)),
                parallel_2(left_pool(heads=2, kv_heads=2, dim=d, vdim=dv, size=size2, pool=P, rot_dims=d // 2))], width=64)
  W = random_weights(cfg, 41)
  toks = rand_tokens(cfg["vocab"], 260, 6)
  ref = oracle_logits(cfg, W, toks)[0]
  outs = []
  for mode in (0, 1):
    n = make_engine(cfg, W, "bfloat16", max_tokens=512, page_size=16)
    n.set_attention_mode(mode)
    got = run_cut(n, 0, toks, [200, 60])
    assert (n.prompt_attention_launches() > 0) == (mode == 0)
    assert row_err(got, ref) < TOL["bfloat16"]
    outs.append(got)
    n.close()
  assert row_err(outs[0], outs[1].astype(np.float64)) < 0.03


# ---- graphs --------------------------------------------------------------------------------------------------------------------
def test_graph_replay_equals_plain_launches():
  cfg = config(MIXED)
  W = random_weights(cfg, 19)
  toks = [rand_tokens(cfg["vocab"], 40, 1), rand_tokens(cfg["vocab"], 33, 2)]
  outs = []
  for graphs in (True, False):
    n = make_engine(cfg, W, "bfloat16", page_size=8)
    n.set_graphs(graphs)
    n.step([0, 1], [toks[0][:10], toks[1][:3]])
    rows = [n.step([0, 1], [toks[0][10 + t:11 + t], toks[1][3 + t:4 + t]])[0] for t in range(30)]
    assert (n.graph_replays() > 20) == graphs
    outs.append(np.stack(rows))
    n.close()
  assert np.array_equal(outs[0], outs[1]), "a replayed decode step must give the bits of the launched one"


# ---- the loader and the entry points -----------------------------------------------------------------------------------------
def write_model_dir(path, cfg, W):
  hdr, blobs, at = {}, [], 0
  for k, t in W.items():
    raw = bf16_bits(t).tobytes()
    hdr[k] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
    blobs.append(raw)
    at += len(raw)
  h = json.dumps(hdr).encode()
  with open(path / "model.safetensors", "wb") as f:
    f.write(struct.pack("<Q", len(h)) + h + b"".join(blobs))
  with open(path / "config.json", "w") as f:
    json.dump(cfg, f)


def test_model_directory_loader_is_strict(tmp_path):
  from xotorch_b200.models import load_model_config, make_native
  cfg = config(MIXED)
  W = random_weights(cfg, 3)
  write_model_dir(tmp_path, cfg, W)
  n = make_native(load_model_config(tmp_path), 0, "float32")
  n.load_dir(tmp_path)
  n.begin_pool(64, 1, 8)
  check(n, cfg, W, rand_tokens(cfg["vocab"], 12, 1), [12], "float32")
  n.close()
  for missing in ("l0.mix.right.i.b", "l1.mix.right.q.conv", "l2.mix.conv.b", "l0.hc2.mix", "l3.canon1", "embed.norm", "l0.mix.left.g", "l2.mix.D"):
    bad = dict(W)
    del bad[missing]
    write_model_dir(tmp_path, cfg, bad)
    with pytest.raises(Exception, match=missing.replace(".", r"\.")):
      make_native(load_model_config(tmp_path), 0, "float32").load_dir(tmp_path)
  for extra, shape in (("l1.mix.left.g", (4, 48)), ("l3.mlp.up", (8, 48)), ("l3.norm2", ()), ("l1.mix.left.q.norm", (8,))):
    bad = dict(W)
    bad[extra] = torch.zeros(shape)                    # a gate the layer type does not have, a feed-forward the layer lacks, norm weights of a weightless norm
    write_model_dir(tmp_path, cfg, bad)
    with pytest.raises(Exception, match=extra.replace(".", r"\.")):
      make_native(load_model_config(tmp_path), 0, "float32").load_dir(tmp_path)


def oracle_greedy(cfg, W, prompt, n_new):
  seq, ids, gaps = list(prompt), [], []
  for _ in range(n_new):
    lg = oracle_logits(cfg, W, np.array(seq))[0][-1]
    top = np.sort(lg)[-2:]
    ids.append(int(np.argmax(lg)))
    gaps.append(float(top[1] - top[0]))
    seq.append(ids[-1])
  return ids, gaps


@pytest.mark.parametrize("dtype,budget", [("float32", 2048), ("bfloat16", 7)])
def test_greedy_generation_through_the_batch_scheduler(dtype, budget):
  from xotorch_b200.scheduler import ContinuousBatch
  cfg = config(MIXED)
  W = random_weights(cfg, 8)
  n = make_engine(cfg, W, dtype)
  events = []
  sched = ContinuousBatch(n, max_requests=3, max_tokens=160, page_size=8, token_budget=budget,
                          on_token=lambda rid, toks, fin: events.append((rid, list(toks), fin)))
  reqs = [(f"r{i}", rand_tokens(cfg["vocab"], L, 70 + i), g) for i, (L, g) in enumerate([(5, 9), (17, 4), (1, 12), (26, 6), (3, 1)])]
  for rid, p, g in reqs[:3]:
    sched.submit(rid, p, g)
  sched.step()
  for rid, p, g in reqs[3:]:
    sched.submit(rid, p, g)                           # joins while others are running
  out = sched.run_until_idle()
  for rid, p, g in reqs:
    ids, gaps = oracle_greedy(cfg, W, p, g)
    assert len(out[rid]) == g
    if out[rid] != ids:                               # after a near tie the continuations differ legitimately
      d = next(i for i in range(g) if out[rid][i] != ids[i])
      assert gaps[d] < (1e-3 if dtype == "float32" else 0.15), f"{rid}: ids leave the oracle's at step {d} with a clear gap {gaps[d]}"
    assert [e[1][0] for e in events if e[0] == rid] == out[rid]
  st = n.cache_stats()
  assert st["pages_free"] == st["pages_total"], "finished requests must give their pages back"
  n.close()


def test_command_line_and_trace_replay_on_a_model_directory(tmp_path, capsys):
  from xotorch_b200.cli import main
  from xotorch_b200.trace_replay import TraceReplayer
  cfg = config(MIXED)
  W = random_weights(cfg, 8)
  write_model_dir(tmp_path, cfg, W)
  prompts = [rand_tokens(cfg["vocab"], 6, 1), rand_tokens(cfg["vocab"], 11, 2)]
  arg = ";".join(",".join(str(int(t)) for t in p) for p in prompts)
  assert main(["generate", "--model", str(tmp_path), "--prompt-ids", arg, "--max-tokens", "5", "--dtype", "float32"]) == 0
  lines = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
  for p, line in zip(prompts, lines):
    ids, gaps = oracle_greedy(cfg, W, p, 5)
    mine = line["ids"]
    if mine != ids:
      d = next(k for k in range(5) if mine[k] != ids[k])
      assert gaps[d] < 1e-3
  out = tmp_path / "out"
  rp = TraceReplayer(tmp_path, "float32", out, max_tokens=128)
  a, b = rand_tokens(cfg["vocab"], 20, 5), rand_tokens(cfg["vocab"], 9, 6)
  rp.run_step({"step": 0, "entries": [{"id": "a", "tokens": a[:14].tolist(), "want": [0, 13]}, {"id": "b", "tokens": b[:3].tolist(), "want": [2]}], "end": []})
  rp.run_step({"step": 1, "entries": [{"id": "a", "tokens": a[14:15].tolist(), "want": [0]}, {"id": "b", "tokens": b[3:4].tolist(), "want": []}], "end": ["b"]})
  rp.run_step({"step": 2, "entries": [{"id": "a", "tokens": a[15:16].tolist(), "want": [0]}], "end": ["a"]})
  rp.close()
  ra, rb = oracle_logits(cfg, W, a)[0], oracle_logits(cfg, W, b)[0]
  s0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(3, -1)
  assert row_err(s0, np.stack([ra[0], ra[13], rb[2]])) < TOL["float32"]
  assert row_err(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1), ra[14:15]) < TOL["float32"]
  assert row_err(np.fromfile(out / "2.f32", dtype="<f4").reshape(1, -1), ra[15:16]) < TOL["float32"]
