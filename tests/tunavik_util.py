"""Helpers of the Tunavik tests: small configurations of the family (attention layers with mixture-of-experts feed-forwards) and
the oracle's logits.  Engines, schedules and the error measure come from layered_util."""
from __future__ import annotations

import copy
from typing import List, Optional, Tuple

import numpy as np
import torch

from tests import tunavik_oracle as to


def moe(experts=6, top=2, ff=12, shared: Optional[int] = 20):
  m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
  if shared:
    m["shared"] = {"ff": shared}
  return m


def attention(heads=4, kv_heads=2, dim=8, vdim=12, scale=None, bias_max=40, temp: Optional[Tuple[float, int]] = (0.5, 16), kv_from=None, mlp=None):
  m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(scale if scale is not None else dim ** -0.5),
       "bias_max": bias_max}
  if temp:
    m["q_temp"] = {"coef": float(temp[0]), "every": int(temp[1])}
  if kv_from is not None:
    m["kv_from"] = int(kv_from)
  return {"type": "attention", "mixer": m, "mlp": mlp}


def config(layers: List[dict], width=48, vocab=80, eps=1e-5, logit_scale: Optional[float] = 0.7, softcap: Optional[float] = 20.0) -> dict:
  c = {"architecture": "Tunavik", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": copy.deepcopy(layers)}
  if logit_scale is not None:
    c["logit_scale"] = logit_scale
  if softcap is not None:
    c["logit_softcap"] = softcap
  return c


def oracle_logits(cfg, weights, tokens, dtype=torch.float64):
  lg, trail = to.forward(cfg, weights, tokens, dtype)
  return lg.double().numpy(), [t.double().numpy() for t in trail]


def close_calls(cfg, weights, tokens, gap=0.15) -> np.ndarray:
  """[T] bool: rows where some router's last chosen logit leads the best one left out by less than `gap`.  With the router's input
  rounded to 16 bits such a row may legitimately choose another expert."""
  gaps = []
  to.forward(cfg, weights, tokens, torch.float64, gaps)
  out = np.zeros(len(tokens), dtype=bool)
  for g in gaps:
    out |= g.numpy() < gap
  return out


def settled_rows(cfg, weights, tokens, dtype: str) -> np.ndarray:
  """[T] bool: the rows a test holds to the tolerance: all of them in float32, all but the close calls in bfloat16"""
  if dtype == "float32":
    return np.ones(len(tokens), dtype=bool)
  return ~close_calls(cfg, weights, tokens)
