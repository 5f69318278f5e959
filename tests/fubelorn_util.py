"""Helpers of the Fubelorn tests: small configurations of the family, random weights that bfloat16 holds exactly, the oracle's
logits.  Engines, schedules and the error measure come from layered_util."""
from __future__ import annotations

import copy
from typing import Dict, List, Optional

import numpy as np
import torch

from tests import fubelorn_oracle as fo


def dense(ff=40):
  return {"kind": "dense", "ff": ff} if ff else None


def left_keep(heads=4, kv_heads=2, dim=8, vdim=12, size=9, keep=3, scale=None):
  return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(scale if scale is not None else dim ** -0.5),
          "mask": {"size": size, "keep_first": keep}}


def left_pool(heads=4, kv_heads=2, dim=8, vdim=12, size=9, pool=4, rot_dims=None, base=100.0, scaling=(4.0, 1.0, 4.0, 32), scale=None):
  m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(scale if scale is not None else dim ** -0.5),
       "mask": {"size": size, "pool": pool}, "rot": {"base": base, "dims": int(dim if rot_dims is None else rot_dims)}}
  if scaling:
    m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
  return m


def right_delta(heads=4, kv_heads=2, dim=8, vdim=6, conv=3):
  return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def right_lstm(heads=3, dim=8, vdim=6, cap=15.0):
  return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def parallel(left=None, right=None, ls=0.8, rs=0.6, ff=40):
  return {"type": "parallel", "mixer": {"left": left or left_keep(), "right": right or right_delta(), "left_scale": ls, "right_scale": rs}, "mlp": dense(ff)}


def parallel_2(left=None, right=None, ls=0.7, rs=0.9, ff=40):
  return {"type": "parallel_2", "mixer": {"left": left or left_pool(), "right": right or right_lstm(), "left_scale": ls, "right_scale": rs}, "mlp": dense(ff)}


def mamba2(heads=4, vdim=6, state=8, groups=2, norm_groups=2, conv=3, ff=40):
  return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}, "mlp": dense(ff)}


def config(layers: List[dict], width=48, vocab=80, eps=1e-5, streams: Optional[int] = 3, taps: Optional[int] = 3, mult=0.7) -> dict:
  c = {"architecture": "Fubelorn", "width": width, "vocab": vocab, "norm": {"eps": eps}, "residual_mult": mult, "layers": copy.deepcopy(layers)}
  if streams:
    c["streams"] = streams
  if taps:
    c["canon"] = {"taps": taps}
  return c


def _r(t: torch.Tensor) -> torch.Tensor:
  return t.to(torch.bfloat16).to(torch.float32)


def random_weights(cfg: dict, seed: int, canon_gain=0.3) -> Dict[str, torch.Tensor]:
  g = torch.Generator().manual_seed(seed)
  D, V, S = cfg["width"], cfg["vocab"], int(cfg.get("streams", 0))
  taps = int((cfg.get("canon") or {}).get("taps", 0))
  n = lambda *shape, dev=1.0, mean=0.0: _r(mean + dev * torch.randn(tuple(shape), generator=g))
  lin = lambda out, inp: n(out, inp, dev=inp ** -0.5)
  W = {"embed": n(V, D), "embed.norm": n(dev=0.1, mean=1.0), "final.norm": n(dev=0.1, mean=1.0), "head": lin(V, D)}
  for i, layer in enumerate(cfg["layers"]):
    p, kind, m = f"l{i}.", layer["type"], layer["mixer"]
    subs = [1] + ([2] if layer.get("mlp") else [])
    for q in subs:
      W[p + f"norm{q}"] = n(dev=0.1, mean=1.0)
      if taps:
        W[p + f"canon{q}"] = n(D, taps, dev=canon_gain * taps ** -0.5)
      if S:
        W[p + f"hc{q}.in"] = _r(0.3 + 0.7 * torch.rand(S, generator=g))
        W[p + f"hc{q}.out"] = _r(0.5 + torch.rand(S, generator=g))
        W[p + f"hc{q}.mix"] = _r(torch.eye(S) + 0.2 * torch.randn(S, S, generator=g))
    if layer.get("mlp"):
      W[p + "mlp.up"], W[p + "mlp.down"] = lin(layer["mlp"]["ff"], D), lin(D, layer["mlp"]["ff"])
    if kind in ("parallel", "parallel_2"):
      a, b = m["left"], m["right"]
      lp, rp = p + "mix.left.", p + "mix.right."
      H, G, d, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
      W[lp + "q"], W[lp + "k"], W[lp + "v"], W[lp + "o"] = lin(H * d, D), lin(G * d, D), lin(G * dv, D), lin(D, H * dv)
      if kind == "parallel_2":
        W[lp + "g"] = lin(H, D)
        H, d, dv = b["heads"], b["dim"], b["vdim"]
        W[rp + "q"], W[rp + "k"], W[rp + "v"], W[rp + "g"], W[rp + "o"] = lin(H * d, D), lin(H * d, D), lin(H * dv, D), lin(H * dv, D), lin(D, H * dv)
        W[rp + "i"], W[rp + "f"] = n(H, D, dev=2.0 * D ** -0.5), n(H, D, dev=2.0 * D ** -0.5)
        W[rp + "i.b"], W[rp + "f.b"] = n(H, dev=1.0), n(H, dev=1.0, mean=2.0)
        W[rp + "norm"] = n(H * dv, dev=0.1, mean=1.0)
      else:
        H, G, d, dv, t = b["heads"], b["kv_heads"], b["dim"], b["vdim"], b["conv"]
        W[rp + "q"], W[rp + "k"], W[rp + "v"], W[rp + "g"], W[rp + "o"] = lin(G * d, D), lin(G * d, D), lin(H * dv, D), lin(H * dv, D), lin(D, H * dv)
        W[rp + "q.conv"], W[rp + "k.conv"], W[rp + "v.conv"] = n(G * d, t, dev=t ** -0.5), n(G * d, t, dev=t ** -0.5), n(H * dv, t, dev=t ** -0.5)
        W[rp + "b"], W[rp + "a"] = lin(H, D), lin(H, D)
        W[rp + "A_log"], W[rp + "dt_bias"] = n(H, dev=0.5), n(H, dev=0.5)
        W[rp + "norm"] = n(dv, dev=0.1, mean=1.0)
    elif kind == "mamba2":
      mp = p + "mix."
      H, dv, N, G, t = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
      inner, C = H * dv, H * dv + 2 * G * N
      W[mp + "in"] = lin(2 * inner + 2 * G * N + H, D)
      W[mp + "conv"], W[mp + "conv.b"] = n(C, t, dev=t ** -0.5), n(C, dev=0.2)
      W[mp + "dt_bias"], W[mp + "A_log"], W[mp + "D"] = n(H, dev=0.5), n(H, dev=0.5), n(H, dev=0.5, mean=1.0)
      W[mp + "norm"], W[mp + "o"] = n(inner, dev=0.1, mean=1.0), lin(D, inner)
    else:
      raise ValueError(kind)
  return W


def oracle_logits(cfg, weights, tokens):
  trail: list = []
  with torch.no_grad():
    lg = fo.forward(cfg, weights, np.asarray(tokens), trail)
  return lg.double().numpy(), [t.double().numpy() for t in trail]
