"""`bench.py --layered`: prefill and decode throughput of the layered engine on Zokuvik-shaped models with random weights, at a
few sizes that resemble a real model's layers, beside the shard engine's Llama decoder of the same width, depth and (to a few
per cent) weight bytes.  One JSON line per size; nothing here touches bench.py's default workload.

`--layered-family bufulorn`: the same for Bufulorn-shaped models (gated delta rule, grouped-query attention with shared keys /
values, dense and mixture-of-experts feed-forwards) beside the closest existing family on the same engine, a Zokuvik model of
the same width and depth whose feed-forward size is chosen so that the weight bytes match.

`--layered-family tunavik`: the same for Tunavik-shaped models (grouped-query attention with learned distance biases, sinks and
shared keys / values; relu^2 experts with a shared expert) beside the closest existing family on the same engine, a Bufulorn
model of attention layers only with the same heads, layer pattern and (to a few per cent) weight bytes.

`--layered-family fubelorn`: the same for Fubelorn-shaped models (two-mixer layers: rotary attention with pooled far blocks + matrix
LSTM, windowed attention that keeps the first tokens + gated delta rule; state-space layers; hyper-connections over four copies of the
stream, input convolutions, gelu feed-forwards) beside the closest existing family on the same engine, a Bufulorn model of gated-delta
and attention layers with dense feed-forwards, of the same width and depth and (to a few per cent) weight bytes.

Timing: every number is the device time of the step(s) (CUDA events on the engine's stream, `last_step_ms` / the ring's own
timer), after warm-up; the weights of every size are larger than L2 from `medium` on, and each prompt step streams all of them.
Roofline denominators come from MEASURED_PEAKS.json (fallback: the profiling recipe's numbers)."""
from __future__ import annotations

import json
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent

# width, layer pattern repeats, attention heads / dn / dr / dv / latent ranks, delta heads x dim, ff, vocab
SIZES = {
  "small": dict(width=1024, repeats=2, heads=8, dim=64, rot_dim=32, vdim=64, kv_rank=256, q_rank=384, dheads=16, ddim=64, ff=4096, vocab=32000),
  "medium": dict(width=2048, repeats=2, heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=512, q_rank=768, dheads=32, ddim=64, ff=8192, vocab=32000),
  "large": dict(width=4096, repeats=2, heads=32, dim=128, rot_dim=64, vdim=128, kv_rank=512, q_rank=1536, dheads=32, ddim=128, ff=14336, vocab=32000),
}
WINDOW, DECAY_RANK = 1024, 64


def zokuvik_config(s: dict):
  def att(kind):
    m = {"heads": s["heads"], "dim": s["dim"], "rot_dim": s["rot_dim"], "vdim": s["vdim"], "kv_rank": s["kv_rank"],
         "rot": {"base": 10000.0, "dims": s["rot_dim"]}, "scale": float((s["dim"] + s["rot_dim"]) ** -0.5)}
    if kind == "latent_attention":
      m["q_rank"] = s["q_rank"]
    else:
      m["mask"] = {"size": WINDOW}
    return {"type": kind, "mixer": m, "mlp": {"kind": "dense", "ff": s["ff"]}}
  layers = []
  for _ in range(s["repeats"]):
    layers += [att("latent_attention"), att("latent_attention_2"),
               {"type": "general_delta", "mixer": {"heads": s["dheads"], "dim": s["ddim"]}, "mlp": {"kind": "dense", "ff": s["ff"]}}]
  cfg = {"architecture": "Zokuvik", "width": s["width"], "vocab": s["vocab"], "norm": {"eps": 1e-6, "groups": 4}, "layers": layers}
  shapes = {f"l{i}.mix.w1": (DECAY_RANK, s["width"]) for i, l in enumerate(layers) if l["type"] == "general_delta"}
  return cfg, shapes


# Bufulorn shapes at the same widths: value heads x size of the delta layers as above, half as many query/key heads; attention
# with 4 query heads per key/value head; 16 experts of a quarter of the dense inner size, 4 per token (as many active weights as
# the dense layers), in 8 groups of which 4 are kept; blocks of 1024 positions
BUFULORN = {
  "small": dict(heads=16, kv_heads=4, dim=64, vdim=64, dheads=16, dkv=8, ddim=64, dvdim=64),
  "medium": dict(heads=16, kv_heads=4, dim=128, vdim=128, dheads=32, dkv=16, ddim=64, dvdim=64),
  "large": dict(heads=32, kv_heads=8, dim=128, vdim=128, dheads=32, dkv=16, ddim=128, dvdim=128),
}
EXPERTS, TOP, GROUPS, KEEP, TAPS = 16, 4, 8, 4, 4


def bufulorn_config(s: dict, b: dict, context: int):
  def att(src, mlp):
    m = {"heads": b["heads"], "kv_heads": b["kv_heads"], "dim": b["dim"], "vdim": b["vdim"], "scale": float(b["dim"] ** -0.5), "softcap": 30.0,
         "mask": {"size": WINDOW}}
    if src is not None:
      m["kv_from"] = src
    return {"type": "attention", "mixer": m, "mlp": mlp}
  dense = {"kind": "dense", "ff": s["ff"]}
  moe = {"kind": "moe", "router": {"experts": EXPERTS, "top": TOP, "groups": {"count": GROUPS, "keep": KEEP}}, "expert": {"ff": s["ff"] // 4}}
  layers = []
  for r in range(s["repeats"]):
    layers += [{"type": "delta", "mixer": {"heads": b["dheads"], "kv_heads": b["dkv"], "dim": b["ddim"], "vdim": b["dvdim"], "conv": TAPS}, "mlp": dense},
               att(None, moe), att(3 * r + 1, dense)]
  cfg = {"architecture": "Bufulorn", "width": s["width"], "vocab": s["vocab"], "max_positions": context, "norm": {"eps": 1e-5}, "layers": layers}
  n_moe = sum(1 for l in layers if l["mlp"]["kind"] == "moe")
  idle = n_moe * (EXPERTS - TOP) * 3 * (s["ff"] // 4) * s["width"] * 2          # bytes of the experts one token does not use
  return cfg, idle


# Tunavik shapes at the same widths: attention heads as the Bufulorn attention layers, per repeat [owner, owner, borrower of the
# second owner], every layer with 16 relu^2 experts (4 per token) and a shared expert of an expert's size; 32 distance buckets up
# to distance 2048, query temperature stepping every 1024 positions.  The Bufulorn model beside it has the same pattern with gated
# experts; the Tunavik experts' inner size is chosen so that (16 + 1) two-matrix experts weigh what 16 three-matrix experts do.
REL_BUCKETS, REL_FAR, TEMP_EVERY = 32, 2048, 1024


def tunavik_config(s: dict, b: dict):
  fb = s["ff"] // 4
  ft = max(64, int(EXPERTS * 3 * fb / ((EXPERTS + 1) * 2)) // 64 * 64)
  moe = {"kind": "moe", "router": {"experts": EXPERTS, "top": TOP}, "expert": {"ff": ft}, "shared": {"ff": ft}}
  def att(src):
    m = {"heads": b["heads"], "kv_heads": b["kv_heads"], "dim": b["dim"], "vdim": b["vdim"], "scale": float(b["dim"] ** -0.5), "bias_max": REL_FAR,
         "q_temp": {"coef": 0.3, "every": TEMP_EVERY}}
    if src is not None:
      m["kv_from"] = src
    return {"type": "attention", "mixer": m, "mlp": moe}
  layers = []
  for r in range(s["repeats"]):
    layers += [att(None), att(None), att(3 * r + 1)]
  cfg = {"architecture": "Tunavik", "width": s["width"], "vocab": s["vocab"], "norm": {"eps": 1e-6}, "logit_scale": 0.7, "logit_softcap": 50.0, "layers": layers}
  shapes = {f"l{i}.mix.rel": (REL_BUCKETS, b["heads"]) for i in range(len(layers))}
  idle = len(layers) * (EXPERTS - TOP) * 2 * ft * s["width"] * 2
  return cfg, shapes, idle, ft


def bufulorn_attention_config(s: dict, b: dict, context: int):
  """Bufulorn layers of the same pattern: causal attention without blocks, 16 gated experts (4 per token, no groups)"""
  fb = s["ff"] // 4
  moe = {"kind": "moe", "router": {"experts": EXPERTS, "top": TOP}, "expert": {"ff": fb}}
  def att(src):
    m = {"heads": b["heads"], "kv_heads": b["kv_heads"], "dim": b["dim"], "vdim": b["vdim"], "scale": float(b["dim"] ** -0.5), "softcap": 30.0}
    if src is not None:
      m["kv_from"] = src
    return {"type": "attention", "mixer": m, "mlp": moe}
  layers = []
  for r in range(s["repeats"]):
    layers += [att(None), att(None), att(3 * r + 1)]
  cfg = {"architecture": "Bufulorn", "width": s["width"], "vocab": s["vocab"], "max_positions": context, "norm": {"eps": 1e-5}, "layers": layers}
  idle = len(layers) * (EXPERTS - TOP) * 3 * fb * s["width"] * 2
  return cfg, idle


# Fubelorn shapes at the same widths, per repeat [rotary pooled attention + matrix LSTM, kept-first attention + gated delta rule,
# state-space layer], every layer with a dense gelu feed-forward; attention heads as the Bufulorn attention layers; the state-space layer
# has 2 * width channels in heads of 64 with 128 states; four copies of the stream, four-tap input convolutions, window 1024 with
# blocks of 64 pooled beyond it resp. the first 4 tokens kept
FUBELORN = {
  "small": dict(lheads=4, ldim=64, lvdim=64, sheads=32, svdim=64, state=128),
  "medium": dict(lheads=8, ldim=64, lvdim=128, sheads=64, svdim=64, state=128),
  "large": dict(lheads=16, ldim=128, lvdim=128, sheads=128, svdim=64, state=128),
}
FUB_STREAMS, FUB_POOL, FUB_KEEP = 4, 64, 4


def fubelorn_config(s: dict, b: dict, f: dict):
  def left(kind):
    m = {"heads": b["heads"], "kv_heads": b["kv_heads"], "dim": b["dim"], "vdim": b["vdim"], "scale": float(b["dim"] ** -0.5)}
    if kind == "parallel":
      m["mask"] = {"size": WINDOW, "keep_first": FUB_KEEP}
    else:
      m["mask"] = {"size": WINDOW, "pool": FUB_POOL}
      m["rot"] = {"base": 500000.0, "dims": b["dim"], "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}
    return m
  dense = {"kind": "dense", "ff": s["ff"]}
  layers = []
  for _ in range(s["repeats"]):
    layers += [{"type": "parallel_2", "mixer": {"left": left("parallel_2"), "right": {"heads": f["lheads"], "dim": f["ldim"], "vdim": f["lvdim"], "gate_cap": 15.0},
                                                 "left_scale": 0.7, "right_scale": 0.7}, "mlp": dense},
               {"type": "parallel", "mixer": {"left": left("parallel"), "right": {"heads": b["dheads"], "kv_heads": b["dkv"], "dim": b["ddim"], "vdim": b["dvdim"], "conv": TAPS},
                                               "left_scale": 0.7, "right_scale": 0.7}, "mlp": dense},
               {"type": "mamba2", "mixer": {"heads": f["sheads"], "vdim": f["svdim"], "state": f["state"], "groups": 1, "norm_groups": 1, "conv": TAPS}, "mlp": dense}]
  return {"architecture": "Fubelorn", "width": s["width"], "vocab": s["vocab"], "norm": {"eps": 1e-6}, "residual_mult": 0.5, "streams": FUB_STREAMS,
          "canon": {"taps": TAPS}, "layers": layers}


def bufulorn_dense_config(s: dict, b: dict, context: int, ff: int):
  """Bufulorn layers with dense feed-forwards only: per repeat [gated delta rule, attention, attention], causal within blocks of 1024"""
  dense = {"kind": "dense", "ff": ff}
  att = {"type": "attention", "mixer": {"heads": b["heads"], "kv_heads": b["kv_heads"], "dim": b["dim"], "vdim": b["vdim"], "scale": float(b["dim"] ** -0.5), "softcap": 30.0,
                                        "mask": {"size": WINDOW}}, "mlp": dense}
  layers = []
  for _ in range(s["repeats"]):
    layers += [{"type": "delta", "mixer": {"heads": b["dheads"], "kv_heads": b["dkv"], "dim": b["ddim"], "vdim": b["dvdim"], "conv": TAPS}, "mlp": dense}, att, att]
  return {"architecture": "Bufulorn", "width": s["width"], "vocab": s["vocab"], "max_positions": context, "norm": {"eps": 1e-5}, "layers": layers}


def peaks():
  p = ROOT / "MEASURED_PEAKS.json"
  if p.exists():
    try:
      d = json.loads(p.read_text())
      return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
    except Exception:
      pass
  return 6650.0, 1590.0, "fallback"


def layered_numbers(s: dict, prompts, decode_ctx: int, decode_batches, steps: int, warmup: int, cfg=None, shapes=None, idle_bytes: int = 0) -> dict:
  """idle_bytes: weights a token does not touch (experts it is not routed to); the FLOP and byte figures count the others"""
  from .layered import LayeredShard
  if cfg is None:
    cfg, shapes = zokuvik_config(s)
  eng = LayeredShard(cfg, 0, "bfloat16")
  eng.set_shard(0, len(cfg["layers"]) - 1, shapes or {})
  eng.init_synthetic(7)
  wbytes = eng.weight_bytes()
  # a prompt step streams the body once + one row of the embedding (and of the position table) per token
  body = wbytes - 2 * s["vocab"] * s["width"] - int(cfg.get("max_positions", 0)) * s["width"] * 2 - idle_bytes
  rng = np.random.default_rng(0)
  out = {"weight_bytes": wbytes, "prefill": {}, "decode": {}}
  max_b = max(decode_batches)
  eng.begin_pool(max(max(prompts), (decode_ctx + steps * 8 + warmup + 8) * max_b) + 64, max_b)   # the decode loop runs warmup + 8 * steps steps
  launches0 = eng.kernel_launches()
  for n in prompts:
    toks = rng.integers(0, s["vocab"], size=n).astype(np.int32)
    ms = []
    for it in range(warmup + steps):
      eng.clear_request(0)
      eng.step([0], [toks])
      if it >= warmup:
        ms.append(eng.last_step_ms())
    t = float(np.median(ms))
    out["prefill"][str(n)] = {"ms": round(t, 3), "tok_s": round(n / t * 1e3, 1), "tflops_weights": round(2 * (body / 2) * n / t / 1e9, 1)}
  for b in decode_batches:
    for sl in range(max_b):
      eng.clear_request(sl)
    ctx = rng.integers(0, s["vocab"], size=(b, decode_ctx)).astype(np.int32)
    eng.step(list(range(b)), [ctx[i] for i in range(b)])
    ms, wall = [], []
    for it in range(warmup + steps * 8):
      t0 = time.perf_counter()
      eng.step(list(range(b)), [rng.integers(0, s["vocab"], size=1).astype(np.int32) for _ in range(b)])
      if it >= warmup:
        wall.append((time.perf_counter() - t0) * 1e3)
        ms.append(eng.last_step_ms())
    t, tw = float(np.median(ms)), float(np.median(wall))
    stream = body + s["vocab"] * s["width"] * 2                      # body + the head matrix per step
    out["decode"][str(b)] = {"ms_device": round(t, 4), "ms_wall": round(tw, 4), "tok_s": round(b / tw * 1e3, 1),
                             "gbs_weights_device": round(stream / t / 1e6, 1)}
  out["kernel_launches"] = eng.kernel_launches() - launches0
  out["tensor_core_launches"] = eng.tensor_core_launches()
  eng.close()
  return out


def llama_numbers(s: dict, target_bytes: int, prompts, decode_ctx: int, steps: int, warmup: int) -> dict:
  """the shard engine on a Llama decoder of the same width and depth; its feed-forward size is chosen so that the weight bytes
  match the layered model's"""
  from .native import NativeShard
  from .synth import ModelShape, hf_config
  D, L, V = s["width"], 3 * s["repeats"], s["vocab"]
  hd = 128 if D >= 2048 else 64
  H = D // hd
  Hkv = max(1, H // 4)
  attn_params = D * (H + 2 * Hkv) * hd + H * hd * D
  per_layer = (target_bytes / 2 - 2 * V * D) / L
  ffn = int(max(512, (per_layer - attn_params) / (3 * D)) // 512 * 512)       # the shard engine wants multiples of 512
  shape = ModelShape("bench", L, D, ffn, H, Hkv, hd, V, max_pos=max(max(prompts), decode_ctx + 4096) + 64)
  eng = NativeShard(hf_config(shape), device=0)
  eng.set_shard(0, L - 1)
  eng.init_synthetic(7)
  rng = np.random.default_rng(0)
  out = {"weight_bytes": eng.weight_bytes(), "ffn": ffn, "prefill": {}, "decode": {}}
  body = out["weight_bytes"] - 2 * V * D
  for n in prompts:
    toks = rng.integers(0, V, size=(1, n)).astype(np.int32)
    ms = []
    for it in range(warmup + steps):
      eng.begin_request(n + 8)
      t0 = time.perf_counter()
      eng.forward(toks, 0)
      if it >= warmup:
        ms.append((time.perf_counter() - t0) * 1e3)
    t = float(np.median(ms))
    out["prefill"][str(n)] = {"ms_wall": round(t, 3), "tok_s": round(n / t * 1e3, 1), "tflops_weights": round(2 * (body / 2) * n / t / 1e9, 1)}
  n_dec = 64
  eng.link_next_local(eng)
  eng.begin_request(decode_ctx + (warmup + steps) * n_dec + 8)
  eng.forward(rng.integers(0, V, size=(1, decode_ctx)).astype(np.int32), 0)
  eng.post_to_next(0)
  ms, step0, pos = [], 0, decode_ctx
  for it in range(warmup + steps):
    eng.ring_launch(n_dec, step0, pos)
    _, t = eng.ring_wait(n_dec)
    step0 += n_dec
    pos += n_dec
    if it >= warmup:
      ms.append(t / n_dec)
  t = float(np.median(ms))
  out["decode"]["1"] = {"ms_device": round(t, 4), "tok_s": round(1e3 / t, 1), "gbs_weights_device": round((body + V * D * 2) / t / 1e6, 1)}
  eng.close()
  return out


def zokuvik_of_bytes(s: dict, target: int) -> dict:
  """the Zokuvik shape of this width and depth whose feed-forward size makes its weight bytes `target`"""
  from .layered import LayeredShard
  def nbytes(ff):
    cfg, shapes = zokuvik_config(dict(s, ff=ff))
    eng = LayeredShard(cfg, 0, "bfloat16")
    eng.set_shard(0, len(cfg["layers"]) - 1, shapes)
    n = eng.weight_bytes()
    eng.close()
    return n
  b0, b1 = nbytes(1024), nbytes(2048)
  ff = int(max(256, 1024 + (target - b0) / ((b1 - b0) / 1024)) // 64 * 64)
  return dict(s, ff=ff)


def run_bufulorn(args, sizes, prompts, hbm, tf, src) -> None:
  for name in sizes:
    s, b = SIZES[name], BUFULORN[name]
    warm = max(3, args.warmup)
    context = max(max(prompts), 1024 + 9 * (args.steps * 8 + warm)) + 64
    cfg, idle = bufulorn_config(s, b, context)
    bu = layered_numbers(s, prompts, decode_ctx=1024, decode_batches=[1, 8], steps=args.steps, warmup=warm, cfg=cfg, idle_bytes=idle)
    zs = zokuvik_of_bytes(s, bu["weight_bytes"])
    z = layered_numbers(zs, prompts, decode_ctx=1024, decode_batches=[1, 8], steps=args.steps, warmup=warm)
    line = {"bench": "layered", "family": "bufulorn", "size": name, "dtype": "bf16", "data": "synthetic", "shape": dict(s, **b), "bufulorn": bu,
            "idle_expert_bytes": idle, "zokuvik_same_size": z, "zokuvik_ff": zs["ff"], "peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": src},
            "frac_of_peak": {
              "bufulorn_decode1_hbm": round(bu["decode"]["1"]["gbs_weights_device"] / hbm, 3),
              "zokuvik_decode1_hbm": round(z["decode"]["1"]["gbs_weights_device"] / hbm, 3),
              **{f"bufulorn_prefill{n}_tensor": round(bu["prefill"][str(n)]["tflops_weights"] / tf, 3) for n in prompts},
              **{f"zokuvik_prefill{n}_tensor": round(z["prefill"][str(n)]["tflops_weights"] / tf, 3) for n in prompts}}}
    print(json.dumps(line), flush=True)


def run_tunavik(args, sizes, prompts, hbm, tf, src) -> None:
  for name in sizes:
    s, b = SIZES[name], BUFULORN[name]
    warm = max(3, args.warmup)
    context = max(max(prompts), 1024 + 9 * (args.steps * 8 + warm)) + 64
    cfg, shapes, idle, ft = tunavik_config(s, b)
    tu = layered_numbers(s, prompts, decode_ctx=1024, decode_batches=[1, 8], steps=args.steps, warmup=warm, cfg=cfg, shapes=shapes, idle_bytes=idle)
    bcfg, bidle = bufulorn_attention_config(s, b, context)
    bu = layered_numbers(s, prompts, decode_ctx=1024, decode_batches=[1, 8], steps=args.steps, warmup=warm, cfg=bcfg, idle_bytes=bidle)
    line = {"bench": "layered", "family": "tunavik", "size": name, "dtype": "bf16", "data": "synthetic", "shape": dict(s, **b, expert_ff=ft), "tunavik": tu,
            "idle_expert_bytes": idle, "bufulorn_same_size": bu, "bufulorn_idle_expert_bytes": bidle,
            "peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": src},
            "frac_of_peak": {
              "tunavik_decode1_hbm": round(tu["decode"]["1"]["gbs_weights_device"] / hbm, 3),
              "bufulorn_decode1_hbm": round(bu["decode"]["1"]["gbs_weights_device"] / hbm, 3),
              **{f"tunavik_prefill{n}_tensor": round(tu["prefill"][str(n)]["tflops_weights"] / tf, 3) for n in prompts},
              **{f"bufulorn_prefill{n}_tensor": round(bu["prefill"][str(n)]["tflops_weights"] / tf, 3) for n in prompts}}}
    print(json.dumps(line), flush=True)


def run_fubelorn(args, sizes, prompts, hbm, tf, src) -> None:
  from .layered import LayeredShard
  for name in sizes:
    s, b, f = SIZES[name], BUFULORN[name], FUBELORN[name]
    warm = max(3, args.warmup)
    context = max(max(prompts), 1024 + 9 * (args.steps * 8 + warm)) + 64
    cfg = fubelorn_config(s, b, f)
    fu = layered_numbers(s, prompts, decode_ctx=1024, decode_batches=[1, 8], steps=args.steps, warmup=warm, cfg=cfg)
    def nbytes(ff):
      eng = LayeredShard(bufulorn_dense_config(s, b, context, ff), 0, "bfloat16")
      eng.set_shard(0, 3 * s["repeats"] - 1, {})
      n = eng.weight_bytes()
      eng.close()
      return n
    b0, b1 = nbytes(1024), nbytes(2048)
    ff = int(max(256, 1024 + (fu["weight_bytes"] - b0) / ((b1 - b0) / 1024)) // 64 * 64)
    bu = layered_numbers(s, prompts, decode_ctx=1024, decode_batches=[1, 8], steps=args.steps, warmup=warm, cfg=bufulorn_dense_config(s, b, context, ff))
    line = {"bench": "layered", "family": "fubelorn", "size": name, "dtype": "bf16", "data": "synthetic", "shape": dict(s, **b, **f), "fubelorn": fu,
            "bufulorn_same_size": bu, "bufulorn_ff": ff, "peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": src},
            "frac_of_peak": {
              "fubelorn_decode1_hbm": round(fu["decode"]["1"]["gbs_weights_device"] / hbm, 3),
              "bufulorn_decode1_hbm": round(bu["decode"]["1"]["gbs_weights_device"] / hbm, 3),
              **{f"fubelorn_prefill{n}_tensor": round(fu["prefill"][str(n)]["tflops_weights"] / tf, 3) for n in prompts},
              **{f"bufulorn_prefill{n}_tensor": round(bu["prefill"][str(n)]["tflops_weights"] / tf, 3) for n in prompts}}}
    print(json.dumps(line), flush=True)


def run(args) -> None:
  hbm, tf, src = peaks()
  sizes = [x for x in (args.layered_sizes or "small,medium,large").split(",") if x]
  prompts = [int(x) for x in (args.layered_prompts or "1024,4096").split(",")]
  if (getattr(args, "layered_family", "") or "zokuvik") == "bufulorn":
    return run_bufulorn(args, sizes, prompts, hbm, tf, src)
  if getattr(args, "layered_family", "") == "tunavik":
    return run_tunavik(args, sizes, prompts, hbm, tf, src)
  if getattr(args, "layered_family", "") == "fubelorn":
    return run_fubelorn(args, sizes, prompts, hbm, tf, src)
  for name in sizes:
    s = SIZES[name]
    z = layered_numbers(s, prompts, decode_ctx=1024, decode_batches=[1, 8], steps=args.steps, warmup=max(3, args.warmup))
    l = llama_numbers(s, z["weight_bytes"], prompts, decode_ctx=1024, steps=args.steps, warmup=max(3, args.warmup))
    line = {"bench": "layered", "size": name, "dtype": "bf16", "data": "synthetic", "shape": s, "zokuvik": z, "llama_same_size": l,
            "peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": src},
            "frac_of_peak": {
              "zokuvik_decode1_hbm": round(z["decode"]["1"]["gbs_weights_device"] / hbm, 3),
              "llama_decode1_hbm": round(l["decode"]["1"]["gbs_weights_device"] / hbm, 3),
              **{f"zokuvik_prefill{n}_tensor": round(z["prefill"][str(n)]["tflops_weights"] / tf, 3) for n in prompts},
              **{f"llama_prefill{n}_tensor": round(l["prefill"][str(n)]["tflops_weights"] / tf, 3) for n in prompts}}}
    print(json.dumps(line), flush=True)
