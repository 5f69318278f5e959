"""The Tunavik family on the layered engine (libxotb200_lm.so) against the plain oracle (tests/tunavik_oracle.py) on small random
models (-m gpu).  The float32 engine is held to the oracle in float64 tightly, the bfloat16 engine loosely; tests ask for the
logits of EVERY row unless they say otherwise, so a wrong key, bucket edge, sink or temperature step at any place shows."""
import json
import struct

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from tests import tunavik_oracle as to
from tests.layered_util import TOL, bf16_bits, make_engine, rand_tokens, row_err, run_cut
from tests.tunavik_util import attention, config, moe, oracle_logits, settled_rows

DTYPES = ["float32", "bfloat16"]

# owners with different shapes, two borrowers of one owner, layers with and without feed-forward / shared expert / temperature
MIXED = [attention(heads=4, kv_heads=2, dim=8, vdim=12, bias_max=40, temp=(0.5, 16), mlp=moe(6, 2, 12, 20)),
         attention(heads=6, kv_heads=3, dim=10, vdim=6, bias_max=15, temp=(1.5, 5), mlp=moe(4, 3, 10, None)),
         attention(heads=4, kv_heads=2, dim=8, vdim=12, bias_max=90, temp=None, kv_from=0, mlp=None),
         attention(heads=4, kv_heads=2, dim=8, vdim=12, bias_max=25, temp=(0.3, 7), kv_from=0, mlp=moe(5, 1, 9, 16)),
         attention(heads=3, kv_heads=1, dim=12, vdim=5, bias_max=33, mlp=moe(3, 3, 7, 11))]
MIXED_BUCKETS = [16, 8, 4, 12, 2]


def check(native, cfg, W, tokens, cuts, dtype, slot=0, tol=None):
  ref, _ = oracle_logits(cfg, W, tokens)
  got = run_cut(native, slot, tokens, cuts)
  ok = settled_rows(cfg, W, tokens, dtype)
  assert ok.mean() > 0.8, "too many rows with a close call between experts: the test would not say much"
  e = row_err(got[ok], ref[ok])
  assert e < (tol or TOL[dtype]), f"{dtype}: rows differ from the oracle, worst relative error {e:.3e}"
  return got


# ---- each mechanism alone ------------------------------------------------------------------------------------------------
SINGLE = {
  "attention": ([attention()], 16),
  "attention_one_kv_head": ([attention(heads=6, kv_heads=1, dim=8, vdim=8)], 16),
  "attention_all_kv_heads": ([attention(heads=5, kv_heads=5, dim=6, vdim=7)], 10),
  "attention_one_head": ([attention(heads=1, kv_heads=1, dim=16, vdim=4)], 16),
  "attention_odd_sizes": ([attention(heads=3, kv_heads=3, dim=5, vdim=3, bias_max=13)], 6),
  "attention_wide_values": ([attention(heads=2, kv_heads=1, dim=40, vdim=72)], 16),
  "attention_many_heads": ([attention(heads=40, kv_heads=8, dim=4, vdim=4)], 16),
  "attention_no_temperature": ([attention(temp=None)], 16),
  "attention_temperature_every_token": ([attention(temp=(0.8, 1))], 16),
  "attention_temperature_steps_of_three": ([attention(temp=(2.0, 3))], 16),
  "attention_two_buckets": ([attention(bias_max=9)], 2),
  "attention_last_bucket_reached_early": ([attention(bias_max=6)], 8),
  "attention_last_bucket_beyond_the_prompt": ([attention(bias_max=5000)], 32),
  "attention_borrowed_keys": ([attention(), attention(bias_max=11, temp=(1.0, 4), kv_from=0)], [16, 6]),
  "no_feed_forward_anywhere": ([attention(), attention(heads=2, kv_heads=2, dim=8, vdim=8)], 8),
  "experts_with_shared": ([attention(mlp=moe(6, 2, 12, 20))], 16),
  "experts_without_shared": ([attention(mlp=moe(6, 2, 12, None))], 16),
  "experts_top_1": ([attention(mlp=moe(5, 1, 16, 8))], 16),
  "experts_all_chosen": ([attention(mlp=moe(4, 4, 8, 8))], 16),
  "experts_odd_sizes": ([attention(heads=3, kv_heads=3, dim=5, vdim=3, mlp=moe(7, 3, 9, 13))], 16),
  "one_expert": ([attention(mlp=moe(1, 1, 24, 24))], 16),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_one_mechanism_models(name, dtype):
  layers, buckets = SINGLE[name]
  cfg = config(layers, width=36 if "odd" in name else 48)
  W = to.random_weights(cfg, 11, buckets)
  n = make_engine(cfg, W, dtype)
  toks = rand_tokens(cfg["vocab"], 41, 3)
  n.set_trace(True)
  ref, trail = oracle_logits(cfg, W, toks)
  got, _ = n.step([0], [toks], want=list(range(len(toks))))
  x = n.read_trace(len(toks))
  for i, t in enumerate(trail):
    assert np.abs(x[i] - t).max() / np.abs(t).max() < (1e-5 if dtype == "float32" else 0.03), f"residual stream after layer {i} differs"
  assert row_err(got, ref) < TOL[dtype]
  n.set_trace(False)
  cut = run_cut(n, 1, toks, [7, 5, 1])               # short portions and single rows: the cache carried between steps
  assert row_err(cut, ref) < TOL[dtype]
  n.close()


@pytest.mark.parametrize("scale,cap", [(None, None), (1.0, 3.0), (2.5, None), (0.2, 50.0)])
def test_logit_scale_and_soft_cap(scale, cap):
  cfg = config([attention(mlp=moe())], logit_scale=scale, softcap=cap)
  W = to.random_weights(cfg, 5)
  n = make_engine(cfg, W, "float32")
  toks = rand_tokens(cfg["vocab"], 9, 1)
  got = check(n, cfg, W, toks, [9], "float32")
  if cap:
    assert np.abs(got).max() <= cap
  _, am = n.step([1], [toks])
  assert am[0] == int(np.argmax(got[-1]))             # the device arg-max is taken on the finished logits
  n.close()


# ---- prefill / decoding / portions -----------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cuts", [[1], [2], [3], [17, 1], [5, 2, 9, 1], [64]])
def test_portions_equal_the_whole_prompt(cuts, dtype):
  cfg = config(MIXED)
  W = to.random_weights(cfg, 2, MIXED_BUCKETS)
  n = make_engine(cfg, W, dtype, page_size=4)
  toks = rand_tokens(cfg["vocab"], 37, 8)
  got = check(n, cfg, W, toks, cuts, dtype)
  n.clear_request(0)
  whole = run_cut(n, 0, toks, [len(toks)])
  assert row_err(got, whole.astype(np.float64)) < (2e-5 if dtype == "float32" else 0.05), "cutting the prompt changes rounding only"
  n.close()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype):
  """300 tokens, all but six decoded one by one: distances pass the last bucket, the temperature steps many times, the keys of a
  decode step are cut into runs over several blocks (the sink must join once, where the runs are merged)"""
  cfg = config([attention(bias_max=120, temp=(0.5, 32), mlp=moe(4, 2, 8, 8)), attention(heads=2, kv_heads=2, dim=8, vdim=8, bias_max=200, temp=(1.0, 100)),
                attention(bias_max=50, kv_from=0, mlp=moe(4, 2, 8, None))], width=32)
  W = to.random_weights(cfg, 21, [16, 32, 8])
  n = make_engine(cfg, W, dtype, max_tokens=400, page_size=16)
  check(n, cfg, W, rand_tokens(cfg["vocab"], 300, 4), [6, 1], dtype)
  n.close()


def test_first_tokens_of_a_sequence():
  cfg = config(MIXED)
  W = to.random_weights(cfg, 9, MIXED_BUCKETS)
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
  W = to.random_weights(cfg, 4, MIXED_BUCKETS)
  n = make_engine(cfg, W, dtype, max_tokens=256, max_requests=5, page_size=4)
  lens = [1, 13, 30, 2, 8]
  seqs = [rand_tokens(cfg["vocab"], L + 6, 50 + i) for i, L in enumerate(lens)]
  refs = [oracle_logits(cfg, W, s)[0] for s in seqs]
  oks = [settled_rows(cfg, W, s, dtype) for s in seqs]
  slots = [3, 0, 4, 1, 2]
  lg, _ = n.step(slots, [s[:L] for s, L in zip(seqs, lens)], want=list(range(sum(lens))))
  at = 0
  for i, L in enumerate(lens):
    assert row_err(lg[at:at + L][oks[i][:L]], refs[i][:L][oks[i][:L]]) < TOL[dtype], f"prompt of request {i}"
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
      if oks[i][lens[i] + t]:
        assert row_err(lg[k:k + 1], refs[i][lens[i] + t:lens[i] + t + 1]) < TOL[dtype], f"request {i}, decoded token {t}"
      assert am[k] == int(np.argmax(lg[k]))
  n.close()


def test_mixed_batch_of_portions_and_decoded_rows():
  cfg = config(MIXED)
  W = to.random_weights(cfg, 6, MIXED_BUCKETS)
  n = make_engine(cfg, W, "float32", page_size=4)
  a, b = rand_tokens(cfg["vocab"], 20, 1), rand_tokens(cfg["vocab"], 26, 2)
  ra, rb = oracle_logits(cfg, W, a)[0], oracle_logits(cfg, W, b)[0]
  n.step([0], [a[:15]])
  lg, _ = n.step([0, 1], [a[15:16], b[:11]], want=list(range(12)))
  assert row_err(lg[:1], ra[15:16]) < TOL["float32"] and row_err(lg[1:], rb[:11]) < TOL["float32"]
  lg, _ = n.step([1, 0], [b[11:26], a[16:17]], want=list(range(16)))
  assert row_err(lg[:15], rb[11:26]) < TOL["float32"] and row_err(lg[15:], ra[16:17]) < TOL["float32"]
  n.close()


# ---- pages and slots that are given back and used again ----------------------------------------------------------------------
def test_freed_pages_and_slots_are_clean_for_the_next_request():
  cfg = config(MIXED)
  W = to.random_weights(cfg, 13, MIXED_BUCKETS)
  n = make_engine(cfg, W, "float32", max_tokens=64, max_requests=2, page_size=4)
  total = n.cache_stats()["pages_total"]
  a, b, c = (rand_tokens(cfg["vocab"], L, s) for L, s in ((29, 1), (18, 2), (31, 3)))
  check(n, cfg, W, a, [9, 1], "float32", slot=0)
  check(n, cfg, W, b, [18], "float32", slot=1)
  assert n.cache_stats()["pages_free"] == total - 8 - 5
  n.clear_request(0)                                  # a's pages go back ...
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


# ---- keys, buckets and sinks made to stand out ---------------------------------------------------------------------------------
def plant(cfg, W):
  """The last two tokens of the vocabulary get embeddings made for each other: the key of the first and every query of the second
  point along one sign vector (the projections are inverted for it; the embeddings are large, so that the position vector hardly
  turns them, and the gain of the embedding norm is divided out), so that this pair's score stands out from all others."""
  m, V = cfg["layers"][0]["mixer"], cfg["vocab"]
  u = torch.tensor([1.0, -1.0] * (m["dim"] // 2), dtype=torch.float64)
  gain = 1.0 + W["embed.norm"].double()
  k_dir = torch.linalg.pinv(W["l0.mix.k"].double()) @ u.repeat(m["kv_heads"]) / gain
  q_dir = torch.linalg.pinv(W["l0.mix.q"].double()) @ u.repeat(m["heads"]) / gain
  W["embed"][V - 2] = (40.0 * k_dir / k_dir.norm()).float()
  W["embed"][V - 1] = (40.0 * q_dir / q_dir.norm()).float()
  W["embed"] = W["embed"].to(torch.bfloat16).to(torch.float32)
  return V - 2, V - 1


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
def test_far_keys_and_page_borders(decode, dtype):
  """One key made to take much of the weight of the last row (sharp scores, planted embeddings): far away (beyond the last bucket's
  start), and on either side of a page border.  Losing it, or reading a neighbour for it, moves the logits by far more than the
  tolerance.  The last 40 rows are decoded one by one when `decode`."""
  V, n_tok = 40, 150
  for name, pos, page in (("far", 3, 16), ("page_first", 64, 64), ("page_last", 63, 64), ("second_token", 1, 8)):
    layer = attention(heads=2, kv_heads=1, dim=16, vdim=12, scale=1.5, bias_max=60, temp=None)
    cfg = config([layer], vocab=V, width=64)
    W = to.random_weights(cfg, 17, 8)
    W["l0.mix.rel"] = (0.2 * W["l0.mix.rel"]).to(torch.bfloat16).to(torch.float32)   # mild biases: a far key can still dominate
    key_tok, query_tok = plant(cfg, W)
    seq = rand_tokens(V - 2, n_tok, 5)
    seq[-1] = query_tok
    without = oracle_logits(cfg, W, seq)[0]
    seq[pos] = key_tok
    ref = oracle_logits(cfg, W, seq)[0]
    gain = np.abs(ref[-1] - without[-1]).max()
    assert gain > 0.5, f"{name}: the planted key does not stand out ({gain})"
    n = make_engine(cfg, W, dtype, max_tokens=256, page_size=page)
    got = run_cut(n, 0, seq, [n_tok - 40, 1] if decode else [n_tok])
    e = row_err(got[-1:], ref[-1:])
    assert e < TOL[dtype], f"{name} ({'decoded' if decode else 'prompt'}): {e:.3e}"
    assert row_err(got, ref) < TOL[dtype]
    n.close()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("buckets,far", [(8, 20), (16, 100), (6, 37), (2, 3), (16, 128)])   # the last: edges that fall exactly on distances 16, 32, 64
def test_bucket_edges(buckets, far, dtype):
  """Every second bucket of the logarithmic half gets a large bias, the others none: a distance counted into the neighbouring bucket
  (one key too early or too late at an edge, in a prompt, in a portion that starts inside the sequence, or in decoding) changes
  that key's weight by e^6."""
  cfg = config([attention(heads=2, kv_heads=1, dim=8, vdim=8, bias_max=far, temp=None)], width=32)
  W = to.random_weights(cfg, 23, buckets)
  rel = torch.zeros(buckets, 2)
  rel[buckets // 2::2] = 6.0
  rel[buckets - 1] = -6.0 if (buckets - 1 - buckets // 2) % 2 else 6.0
  W["l0.mix.rel"] = rel
  toks = rand_tokens(cfg["vocab"], far + 40, 3)
  n = make_engine(cfg, W, dtype, max_tokens=512, page_size=16)
  check(n, cfg, W, toks, [len(toks)], dtype, slot=0)
  check(n, cfg, W, toks, [far // 2 + 3, 19, 1], dtype, slot=1)
  n.close()


@pytest.mark.parametrize("dtype", DTYPES)
def test_sinks_of_every_size(dtype):
  """head 0 has a sink that takes nearly everything, head 1 one that takes nearly nothing, head 2 an ordinary one: a sink that is
  left out, scaled, biased or counted per key run shows on one head or another (prompt, and decoding over several key runs)"""
  cfg = config([attention(heads=3, kv_heads=1, dim=8, vdim=8, bias_max=30, mlp=None)], width=32)
  W = to.random_weights(cfg, 29, 8)
  W["l0.mix.sink"] = torch.tensor([9.0, -9.0, 1.5])
  toks = rand_tokens(cfg["vocab"], 200, 7)
  without = dict(W)
  without["l0.mix.sink"] = torch.full((3,), -80.0)
  assert row_err(oracle_logits(cfg, without, toks)[0], oracle_logits(cfg, W, toks)[0]) > 0.05, "the sinks must matter"
  n = make_engine(cfg, W, dtype, max_tokens=512, page_size=16)
  check(n, cfg, W, toks, [len(toks)], dtype, slot=0)
  check(n, cfg, W, toks, [150, 1], dtype, slot=1)
  n.close()


def test_temperature_follows_the_position_not_the_portion():
  """a strong temperature that steps every 8 positions: a portion that starts at position 13 must scale its queries by the
  positions in the sequence, not by those in the portion"""
  cfg = config([attention(heads=2, kv_heads=2, dim=8, vdim=8, scale=0.5, temp=(3.0, 8))], width=32)
  W = to.random_weights(cfg, 31, 8)
  toks = rand_tokens(cfg["vocab"], 60, 9)
  plain = config([attention(heads=2, kv_heads=2, dim=8, vdim=8, scale=0.5, temp=None)], width=32)
  assert row_err(oracle_logits(plain, W, toks)[0], oracle_logits(cfg, W, toks)[0]) > 0.05, "the temperature must matter"
  n = make_engine(cfg, W, "float32", page_size=8)
  check(n, cfg, W, toks, [13, 20, 1], "float32")
  n.close()


def test_borrowed_keys_are_the_owner_layers_normed_keys():
  """a layer that reads another layer's keys/values sees them as the owner's cache holds them (after the owner's key norm), with its
  own queries, biases, sink and temperature: with a large key-norm weight on one channel of the owner a wrong source would show"""
  cfg = config([attention(heads=2, kv_heads=2, dim=8, vdim=8), attention(heads=4, kv_heads=1, dim=6, vdim=6, mlp=moe(3, 1, 8, 8)),
                attention(heads=2, kv_heads=2, dim=8, vdim=8, bias_max=12, temp=(1.0, 6), kv_from=0)], width=32)
  W = to.random_weights(cfg, 5, [16, 8, 4])
  W["l0.mix.k.norm"][3] = 6.0
  n = make_engine(cfg, W, "float32", page_size=4)
  check(n, cfg, W, rand_tokens(cfg["vocab"], 45, 2), [19, 1], "float32")
  n.close()


# ---- several shards ----------------------------------------------------------------------------------------------------------
def test_two_shards_hand_over_the_residual_stream():
  cfg = config(MIXED)
  W = to.random_weights(cfg, 31, MIXED_BUCKETS)
  a = make_engine(cfg, W, "float32", start=0, end=3)          # the borrowing layers 2 and 3 stay with their owner, layer 0
  b = make_engine(cfg, W, "float32", start=4, end=4)
  toks = rand_tokens(cfg["vocab"], 19, 7)
  ref = oracle_logits(cfg, W, toks)[0]
  hid = a.step([0], [toks[:12]])
  lg, _ = b.step([0], [hid], want=list(range(12)))
  assert row_err(lg, ref[:12]) < TOL["float32"]
  hid = a.step([0], [toks[12:]])
  lg, _ = b.step([0], [hid], want=list(range(7)))
  assert row_err(lg, ref[12:]) < TOL["float32"]
  a.close()
  b.close()
  with pytest.raises(Exception, match="earlier layer of this shard"):
    make_engine(cfg, W, "float32", start=2, end=4)


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
  W = to.random_weights(cfg, 3, MIXED_BUCKETS)
  write_model_dir(tmp_path, cfg, W)
  n = make_native(load_model_config(tmp_path), 0, "float32")
  n.load_dir(tmp_path)
  n.begin_pool(64, 1, 8)
  check(n, cfg, W, rand_tokens(cfg["vocab"], 12, 1), [12], "float32")
  n.close()
  for missing in ("l0.mix.sink", "l1.mlp.e3.up", "l1.mlp.router.b", "l0.mlp.shared.down", "l3.mix.o.b", "embed.norm", "l4.mix.k.norm"):
    bad = dict(W)
    del bad[missing]
    write_model_dir(tmp_path, cfg, bad)
    with pytest.raises(Exception, match=missing.replace(".", r"\.")):
      make_native(load_model_config(tmp_path), 0, "float32").load_dir(tmp_path)
  for extra, shape in (("l2.mix.k", (16, 48)), ("l1.mlp.shared.up", (8, 48)), ("l0.mlp.e0.gate", (12, 48)), ("final.norm.b", (48,))):
    bad = dict(W)
    bad[extra] = torch.zeros(*shape)                   # a borrower's keys, a shared expert the config does not have, a gate matrix, a norm bias
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
  W = to.random_weights(cfg, 8, MIXED_BUCKETS)
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


def test_command_line_generates_from_a_model_directory(tmp_path, capsys):
  from xotorch_b200.cli import main
  cfg = config(MIXED)
  W = to.random_weights(cfg, 8, MIXED_BUCKETS)
  write_model_dir(tmp_path, cfg, W)
  prompts = [rand_tokens(cfg["vocab"], 6, 1), rand_tokens(cfg["vocab"], 11, 2)]
  arg = ";".join(",".join(str(int(t)) for t in p) for p in prompts)
  assert main(["generate", "--model", str(tmp_path), "--prompt-ids", arg, "--max-tokens", "5", "--dtype", "float32"]) == 0
  lines = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
  for p, line in zip(prompts, lines):
    ids, gaps = oracle_greedy(cfg, W, p, 5)
    if line["ids"] != ids:
      d = next(i for i in range(5) if line["ids"][i] != ids[i])
      assert gaps[d] < 1e-3


def test_trace_replay_of_a_model_directory(tmp_path):
  """the token-trace replayer on a model directory: prompts in one batch, then decoding together, one request ending early"""
  from xotorch_b200.trace_replay import TraceReplayer
  cfg = config(MIXED)
  W = to.random_weights(cfg, 15, MIXED_BUCKETS)
  model, out = tmp_path / "m", tmp_path / "o"
  model.mkdir()
  write_model_dir(model, cfg, W)
  a, b = rand_tokens(cfg["vocab"], 22, 1), rand_tokens(cfg["vocab"], 9, 2)
  ra, rb = oracle_logits(cfg, W, a)[0], oracle_logits(cfg, W, b)[0]
  rp = TraceReplayer(model, "float32", out, max_tokens=64)
  rp.run_step({"step": 0, "entries": [{"id": "a", "tokens": a[:18].tolist(), "want": [0, 17]}, {"id": "b", "tokens": b[:8].tolist(), "want": [7]}], "end": []})
  rp.run_step({"step": 1, "entries": [{"id": "a", "tokens": [int(a[18])], "want": [0]}, {"id": "b", "tokens": [int(b[8])], "want": [0]}], "end": ["b"]})
  rp.run_step({"step": 2, "entries": [{"id": "a", "tokens": a[19:22].tolist(), "want": []}], "end": ["a"]})
  V = cfg["vocab"]
  s0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V)
  s1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(-1, V)
  assert row_err(s0, np.stack([ra[0], ra[17], rb[7]])) < TOL["float32"]
  assert row_err(s1, np.stack([ra[18], rb[8]])) < TOL["float32"]
  assert not (out / "2.f32").exists()
  rp.close()


def test_inference_engine_serves_a_model_directory(tmp_path):
  """`B200ShardInferenceEngine` (the engine interface the node drives) on a model split over two shards, two request ids
  interleaved: ensure_shard -> registry -> LayeredShard, the position protocol of infer_tensor, sample(temp 0)"""
  import asyncio
  from xotorch_b200.inference.b200_engine import B200ShardInferenceEngine, LocalDirDownloader
  from xotorch_b200.inference.shard import Shard
  cfg = config(MIXED)
  W = to.random_weights(cfg, 27, MIXED_BUCKETS)
  write_model_dir(tmp_path, cfg, W)
  n = len(cfg["layers"])
  first, last = Shard("m", 0, 3, n), Shard("m", 4, n - 1, n)          # the borrowers (layers 2, 3) stay with their owner
  prompts = {"a": rand_tokens(cfg["vocab"], 9, 1), "b": rand_tokens(cfg["vocab"], 21, 2)}

  async def run():
    e1 = B200ShardInferenceEngine(LocalDirDownloader({"m": tmp_path}), device=0, max_concurrent_requests=2, max_total_len=64)
    e2 = B200ShardInferenceEngine(LocalDirDownloader({"m": tmp_path}), device=0, max_concurrent_requests=2, max_total_len=64)
    out, state, data = {r: [] for r in prompts}, {r: None for r in prompts}, {r: p.reshape(1, -1).astype(np.int64) for r, p in prompts.items()}
    for _ in range(4):
      for r in prompts:                               # the two requests take turns, token by token
        hid, st = await e1.infer_tensor(r, first, data[r], state[r])
        assert hid.ndim == 3 and hid.shape[2] == cfg["width"]
        logits, st2 = await e2.infer_tensor(r, last, hid, state[r])
        tok = await e2.sample(logits, temp=0.0)
        out[r].append(int(tok[0, 0]))
        state[r] = st2
        data[r] = tok.reshape(1, 1).astype(np.int64)
    return out

  out = asyncio.run(run())
  for r, p in prompts.items():
    ids, gaps = oracle_greedy(cfg, W, p, 4)
    if out[r] != ids:
      d = next(i for i in range(4) if out[r][i] != ids[i])
      assert gaps[d] < 0.15, f"{r}: ids leave the oracle's at step {d} with a clear gap"


# ---- decode steps replayed from CUDA graphs ----------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
def test_graph_replay_of_decode_steps_changes_nothing(dtype):
  cfg = config(MIXED)
  W = to.random_weights(cfg, 19, MIXED_BUCKETS)
  seqs = [rand_tokens(cfg["vocab"], 300, 40 + i) for i in range(3)]
  starts = [240, 3, 17]

  def run(graphs):
    n = make_engine(cfg, W, dtype, max_tokens=1000, max_requests=3, page_size=8)
    n.set_graphs(graphs)
    n.step([0, 1, 2], [s[:k] for s, k in zip(seqs, starts)])
    out, live = [], [0, 1, 2]
    for t in range(40):
      if t == 25:
        live = [0, 2]
        n.clear_request(1)
      lg, _ = n.step(live, [seqs[i][starts[i] + t:starts[i] + t + 1] for i in live])
      out.append(lg)
    replays = n.graph_replays()
    n.close()
    return out, replays

  plain, r0 = run(False)
  replayed, r1 = run(True)
  assert r0 == 0 and r1 >= 30
  for a, b in zip(plain, replayed):
    assert np.array_equal(a, b)
  ref = oracle_logits(cfg, W, seqs[0][:280])[0]
  got = np.stack([x[0] for x in replayed])
  assert row_err(got, ref[240:280]) < TOL[dtype]


# ---- sizes the tensor-core paths take ----------------------------------------------------------------------------------------
def test_prompt_kernels_on_aligned_sizes_equal_the_plain_ones():
  """sizes that are multiples of 8 and prompts of hundreds of rows: the bf16 engine runs its products, its prompt attention (with
  the learned biases staged per tile and the sink folded in at the end) and its experts (grouped products, relu^2 in the epilogue)
  on the tensor cores there; the results must agree with the plain kernels on the same 16-bit operands and with the oracle"""
  layers = [attention(heads=4, kv_heads=2, dim=16, vdim=24, bias_max=70, temp=(0.5, 50), mlp=moe(8, 2, 32, 48)),
            attention(heads=4, kv_heads=2, dim=16, vdim=24, bias_max=250, temp=None, kv_from=0, mlp=moe(4, 2, 40, None)),
            attention(heads=2, kv_heads=2, dim=32, vdim=64, bias_max=128, temp=(1.0, 128), mlp=moe(6, 3, 16, 24))]
  cfg = config(layers, width=64, vocab=136)
  W = to.random_weights(cfg, 12, [16, 32, 8])
  n = make_engine(cfg, W, "bfloat16", max_tokens=1400, max_requests=3, page_size=32)
  a, b = rand_tokens(cfg["vocab"], 300, 9), rand_tokens(cfg["vocab"], 150, 10)
  ra, rb = oracle_logits(cfg, W, a)[0], oracle_logits(cfg, W, b)[0]
  before, flash_before = n.tensor_core_launches(), n.prompt_attention_launches()
  lg1, _ = n.step([0, 1], [a[:200], b], want=list(range(350)))          # a's first 200 rows and all of b in one batch
  lg2, _ = n.step([0], [a[200:]], want=list(range(100)))               # the rest of a starts far inside the sequence
  assert n.tensor_core_launches() > before and n.prompt_attention_launches() > flash_before
  tc_a = np.concatenate([lg1[:200], lg2])
  oka, okb = settled_rows(cfg, W, a, "bfloat16"), settled_rows(cfg, W, b, "bfloat16")
  assert oka.mean() > 0.8 and okb.mean() > 0.8
  assert row_err(tc_a[oka], ra[oka]) < TOL["bfloat16"] and row_err(lg1[200:][okb], rb[okb]) < TOL["bfloat16"]
  # three requests decode together: grouped expert products inside decode steps that are captured and replayed as CUDA graphs
  c = rand_tokens(cfg["vocab"], 12, 11)
  n.step([2], [c[:4]])
  a2, b2 = np.concatenate([a, a[:8]]), np.concatenate([b, b[:8]])
  ra2, rb2, rc = oracle_logits(cfg, W, a2)[0], oracle_logits(cfg, W, b2)[0], oracle_logits(cfg, W, c)[0]
  ok2 = [settled_rows(cfg, W, s, "bfloat16") for s in (a2, b2, c)]
  replays = n.graph_replays()
  for t in range(8):
    lg, _ = n.step([0, 1, 2], [a2[300 + t:301 + t], b2[150 + t:151 + t], c[4 + t:5 + t]])
    keep = np.array([ok2[0][300 + t], ok2[1][150 + t], ok2[2][4 + t]])
    assert row_err(lg[keep], np.stack([ra2[300 + t], rb2[150 + t], rc[4 + t]])[keep]) < TOL["bfloat16"], f"decoded token {t}"
  assert n.graph_replays() - replays >= 5
  n.clear_request(2)
  n.set_gemm_mode(1)
  n.set_attention_mode(1)
  fma = run_cut(n, 2, a, [200, 100])
  assert row_err(fma[oka], ra[oka]) < TOL["bfloat16"]
  assert row_err(tc_a[oka], fma.astype(np.float64)[oka]) < 0.05, "16-bit operands and fp32 accumulation in both"
  n.close()


# ---- other shapes, drawn at random ---------------------------------------------------------------------------------------------
def random_model(seed):
  """a model whose sizes, layer order, bucket counts, temperatures and routing are drawn from ranges that include multiples of 8
  (tensor-core kernels) and odd values (plain kernels); borrowing layers point at any earlier owner, several may share one"""
  r = np.random.default_rng(seed)
  pick = lambda *xs: xs[int(r.integers(len(xs)))]
  aligned = seed % 2 == 0
  width = pick(64, 96, 160) if aligned else pick(40, 52, 100)
  layers, owners, buckets = [], [], []
  for i in range(int(r.integers(3, 7))):
    mlp = pick(None, "moe", "moe", "moe")
    if mlp == "moe":
      E = pick(3, 4, 6, 12)
      mlp = moe(E, int(r.integers(1, min(4, E) + 1)), pick(16, 40) if aligned else pick(9, 20), pick(None, 24, 56) if aligned else pick(None, 13, 30))
    temp = pick(None, (0.5, 64), (1.0, 10), (0.25, 1))
    far = pick(20, 64, 150, 1000)
    buckets.append(pick(2, 4, 8, 16, 32))
    if owners and r.random() < 0.4:
      src = pick(*owners)
      m = layers[src]["mixer"]
      layers.append(attention(heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"], bias_max=far, temp=temp, kv_from=src, mlp=mlp))
    else:
      G = pick(1, 2, 3)
      H = G * pick(1, 2, 4)
      dk, dv = (pick(16, 40, 80), pick(8, 24, 96)) if aligned else (pick(5, 12, 33), pick(3, 10, 20))
      layers.append(attention(heads=H, kv_heads=G, dim=dk, vdim=dv, bias_max=far, temp=temp, mlp=mlp))
      owners.append(i)
  return config(layers, width=width, vocab=pick(50, 131), logit_scale=pick(None, 0.5, 2.0), softcap=pick(None, 10.0, 40.0)), buckets


def row_errors(got, ref):
  d = got.astype(np.float64) - ref
  d = d - d.mean(axis=-1, keepdims=True)
  r = ref - ref.mean(axis=-1, keepdims=True)
  return np.sqrt((d * d).mean(-1)) / np.sqrt((r * r).mean(-1) + 1e-30)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed", range(8))
def test_models_drawn_at_random(seed, dtype):
  """whole prompts (one long enough for the tensor-core kernels next to a short one), then decoding together, then a portion.
  float32: every row within the tolerance.  bfloat16: rows where two router logits lie closer than the rounding of the router's
  input may choose another expert legitimately and are left out.  Of the others a few may still leave the tolerance, by little: the
  closing norm scales a feed-forward output to unit size however small it is, so a row whose chosen experts are barely active has
  its 16-bit rounding magnified, and later rows read that row's keys.  The typical row stays tight."""
  cfg, buckets = random_model(seed)
  W = to.random_weights(cfg, 100 + seed, buckets)
  n = make_engine(cfg, W, dtype, max_tokens=800, max_requests=3, page_size=16)
  a, b = rand_tokens(cfg["vocab"], 180, seed), rand_tokens(cfg["vocab"], 30, seed + 50)
  ra, rb = oracle_logits(cfg, W, a)[0], oracle_logits(cfg, W, b)[0]
  oka, okb = settled_rows(cfg, W, a, dtype), settled_rows(cfg, W, b, dtype)
  errs, keep = [], []
  lg, _ = n.step([2, 0], [a[:140], b[:9]], want=list(range(149)))
  errs += [row_errors(lg[:140], ra[:140]), row_errors(lg[140:], rb[:9])]
  keep += [oka[:140], okb[:9]]
  for t in range(21):
    lg, _ = n.step([0, 2], [b[9 + t:10 + t], a[140 + t:141 + t]])
    errs += [row_errors(lg[:1], rb[9 + t:10 + t]), row_errors(lg[1:], ra[140 + t:141 + t])]
    keep += [okb[9 + t:10 + t], oka[140 + t:141 + t]]
  lg, _ = n.step([2], [a[161:]], want=list(range(19)))               # a portion of 19 rows after decoding
  errs.append(row_errors(lg, ra[161:]))
  keep.append(oka[161:])
  e, keep = np.concatenate(errs), np.concatenate(keep)
  n.close()
  assert keep.mean() > 0.6, "too many close calls between experts: the test would not say much"
  if dtype == "float32":
    assert e.max() < TOL[dtype], json.dumps(cfg["layers"])
  else:
    over = (e[keep] > TOL[dtype]).mean()
    assert over <= 0.1 and e[keep].max() < 4 * TOL[dtype], f"{(e[keep] > TOL[dtype]).sum()} of {keep.sum()} rows, worst {e[keep].max():.3f}: " + json.dumps(cfg["layers"])
  assert np.median(e) < 0.3 * TOL[dtype]
