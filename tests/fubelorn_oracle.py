"""Plain restatement of the Fubelorn design: whole sequences, no cache, no batching, one function per mechanism, float64 by default.
It shares no code with the product path (xotorch_b200/, csrc/); the GPU tests compare the engine with it.

A model is (config, weights): `config` the dict of config.json, `weights` name -> torch tensor.  A layer reads `streams` copies of
the residual stream through hyper-connections; every sublayer input passes a scalar-weight RMS norm and a causal per-channel
convolution that is ADDED to it; the mixers are two-branch ("parallel": windowed attention that keeps the first tokens + gated
delta rule; "parallel_2": rotary windowed attention with pooled far blocks + matrix-memory LSTM) or a Mamba-2 state-space layer."""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

DT = torch.float64


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
  return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def causal_conv(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
  """x [T, C], w [C, taps] (last column = the current token); zeros before the start"""
  T, taps = x.shape[0], w.shape[1]
  out = torch.zeros_like(x)
  for j in range(taps):
    back = taps - 1 - j
    if back < T:
      out[back:] += x[: T - back] * w[:, j]
  if bias is not None:
    out = out + bias
  return out


def silu(x):
  return x * torch.sigmoid(x)


def softplus(x):
  return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def gelu_erf(x):
  return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))


# ---- attention branches ------------------------------------------------------------------------------------------------------
def rotary_frequencies(rot: dict) -> torch.Tensor:
  dims, base = int(rot["dims"]), float(rot["base"])
  f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=DT)
  sc = rot.get("scaling")
  if sc:
    factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
    out = []
    for fi in f.tolist():
      wl = 2 * math.pi / fi
      if wl < orig / high:
        out.append(fi)
      elif wl > orig / low:
        out.append(fi / factor)
      else:
        s = (orig / wl - low) / (high - low)
        out.append((1 - s) * fi / factor + s * fi)
    f = torch.tensor(out, dtype=DT)
  return f


def rotate_half_layout(x: torch.Tensor, pos: torch.Tensor, f: torch.Tensor, dims: int) -> torch.Tensor:
  """x [T, heads, d]; entry i < dims/2 is paired with i + dims/2; the rest passes"""
  half = dims // 2
  ang = pos.to(DT)[:, None] * f[None, :]
  c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
  u, v = x[..., :half], x[..., half:dims]
  return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def attend(q, k, v, visible, scale):
  """q [T, H, d], k [S, G, d], v [S, G, dv], visible [T, S] bool -> [T, H, dv]"""
  H, G = q.shape[1], k.shape[1]
  rep = H // G
  out = torch.zeros(q.shape[0], H, v.shape[-1], dtype=q.dtype)
  for a in range(H):
    g = a // rep
    s = (q[:, a] @ k[:, g].T) * scale
    s = s.masked_fill(~visible, float("-inf"))
    out[:, a] = torch.softmax(s, dim=-1) @ v[:, g]
  return out


def attention_keep_first(h, W, m, eps):
  """no rotation; weightless RMS norm of every query / key head; window `size` plus the first `keep_first` tokens"""
  T = h.shape[0]
  H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
  q = rms_unit((h @ W["q"].T).view(T, H, d), eps)
  k = rms_unit((h @ W["k"].T).view(T, G, d), eps)
  v = (h @ W["v"].T).view(T, G, dv)
  size, keep = int(m["mask"]["size"]), int(m["mask"].get("keep_first", 0))
  i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
  vis = (j <= i) & ((i - j < size) | (j < keep))
  o = attend(q, k, v, vis, float(m["scale"]))
  return o.reshape(T, H * dv) @ W["o"].T


def attention_pooled(h, W, m, eps):
  """rotary (rotate-half, frequency scaling); window `size`; every block of `pool` tokens that lies wholly before a row's window is
  seen as ONE key / value (the means over the block); one sigmoid gate per head"""
  T = h.shape[0]
  H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
  q = (h @ W["q"].T).view(T, H, d)
  k = (h @ W["k"].T).view(T, G, d)
  v = (h @ W["v"].T).view(T, G, dv)
  if m.get("rot"):
    f, dims, pos = rotary_frequencies(m["rot"]), int(m["rot"]["dims"]), torch.arange(T)
    q, k = rotate_half_layout(q, pos, f, dims), rotate_half_layout(k, pos, f, dims)
  size, P = int(m["mask"]["size"]), int(m["mask"].get("pool", 0))
  i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
  vis = (j <= i) & (i - j < size)
  nb = T // P if P > 0 else 0
  if nb > 0:
    kb = k[: nb * P].view(nb, P, G, d).mean(1)
    vb = v[: nb * P].view(nb, P, G, dv).mean(1)
    b = torch.arange(nb)[None, :]
    visb = (b * P + P - 1) <= (i - size)
    k, v, vis = torch.cat([kb, k]), torch.cat([vb, v]), torch.cat([visb, vis], dim=1)
  o = attend(q, k, v, vis, float(m["scale"]))
  gate = torch.sigmoid(h @ W["g"].T)                       # [T, H]
  o = o * gate[:, :, None]
  return o.reshape(T, H * dv) @ W["o"].T


# ---- recurrent branches --------------------------------------------------------------------------------------------------------
def gated_delta_rule(h, W, m, eps):
  T = h.shape[0]
  H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
  q = silu(causal_conv(h @ W["q"].T, W["q.conv"])).view(T, G, d)
  k = silu(causal_conv(h @ W["k"].T, W["k.conv"])).view(T, G, d)
  v = silu(causal_conv(h @ W["v"].T, W["v.conv"])).view(T, H, dv)
  q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
  k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
  beta = torch.sigmoid(h @ W["b"].T)
  g = torch.exp(-torch.exp(W["A_log"]) * softplus(h @ W["a"].T + W["dt_bias"]))
  gate = silu(h @ W["g"].T).view(T, H, dv)
  rep = H // G
  out = torch.zeros(T, H, dv, dtype=h.dtype)
  for a in range(H):
    S = torch.zeros(d, dv, dtype=h.dtype)
    for t in range(T):
      kt, qt = k[t, a // rep], q[t, a // rep]
      S = g[t, a] * S
      u = beta[t, a] * (v[t, a] - S.T @ kt)
      S = S + torch.outer(kt, u)
      out[t, a] = S.T @ qt
  out = rms_unit(out, eps) * W["norm"] * gate
  return out.reshape(T, H * dv) @ W["o"].T


def matrix_lstm(h, W, m, eps):
  T = h.shape[0]
  H, d, dv, cap = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["gate_cap"])
  q = (h @ W["q"].T).view(T, H, d) * d ** -0.5
  k = (h @ W["k"].T).view(T, H, d)
  v = (h @ W["v"].T).view(T, H, dv)
  ig = cap * torch.tanh((h @ W["i"].T + W["i.b"]) / cap)
  fg = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ W["f"].T + W["f.b"]) / cap))
  out = torch.zeros(T, H, dv, dtype=h.dtype)
  for a in range(H):
    S, n, mx = torch.zeros(d, dv, dtype=h.dtype), torch.zeros(d, dtype=h.dtype), torch.zeros((), dtype=h.dtype)
    for t in range(T):
      m_new = torch.maximum(fg[t, a] + mx, ig[t, a])
      decay, inp = torch.exp(fg[t, a] + mx - m_new), torch.exp(ig[t, a] - m_new)
      S = decay * S + inp * torch.outer(k[t, a], v[t, a])
      n = decay * n + inp * k[t, a]
      mx = m_new
      den = torch.maximum(torch.abs(n @ q[t, a]), torch.exp(-mx)) + 1e-6
      out[t, a] = (S.T @ q[t, a]) / den
  out = rms_unit(out, eps).reshape(T, H * dv) * W["norm"] * torch.sigmoid(h @ W["g"].T)
  return out @ W["o"].T


def mamba2(h, W, m, eps):
  T = h.shape[0]
  H, dv, N, G, NG = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"]), int(m["norm_groups"])
  inner = H * dv
  p = h @ W["in"].T
  z, xbc, dt = p[:, :inner], p[:, inner: 2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N:]
  xbc = silu(causal_conv(xbc, W["conv"], W["conv.b"]))
  x, B, Cm = xbc[:, :inner].view(T, H, dv), xbc[:, inner: inner + G * N].view(T, G, N), xbc[:, inner + G * N:].view(T, G, N)
  dt = softplus(dt + W["dt_bias"])
  A = -torch.exp(W["A_log"])
  rep = H // G
  y = torch.zeros(T, H, dv, dtype=h.dtype)
  for a in range(H):
    S = torch.zeros(N, dv, dtype=h.dtype)
    for t in range(T):
      S = torch.exp(A[a] * dt[t, a]) * S + dt[t, a] * torch.outer(B[t, a // rep], x[t, a])
      y[t, a] = S.T @ Cm[t, a // rep] + W["D"][a] * x[t, a]
  y = y.reshape(T, inner) * silu(z)
  y = rms_unit(y.view(T, NG, inner // NG), eps).reshape(T, inner) * W["norm"]
  return y @ W["o"].T


def parallel_mixer(kind, h, W, m, eps):
  left = {k[5:]: v for k, v in W.items() if k.startswith("left.")}
  right = {k[6:]: v for k, v in W.items() if k.startswith("right.")}
  if kind == "parallel":
    a, b = attention_keep_first(h, left, m["left"], eps), gated_delta_rule(h, right, m["right"], eps)
  else:
    a, b = attention_pooled(h, left, m["left"], eps), matrix_lstm(h, right, m["right"], eps)
  return float(m["left_scale"]) * a + float(m["right_scale"]) * b


def mixer(kind, h, W, m, eps):
  if kind in ("parallel", "parallel_2"):
    return parallel_mixer(kind, h, W, m, eps)
  if kind == "mamba2":
    return mamba2(h, W, m, eps)
  raise ValueError(kind)


def feed_forward(h, W):
  return gelu_erf(h @ W["up"].T) @ W["down"].T


# ---- the block -------------------------------------------------------------------------------------------------------------------
def sublayer_input(u, g, eps, canon_w):
  h = rms_unit(u, eps) * g
  if canon_w is not None:
    h = h + causal_conv(h, canon_w)
  return h


def sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
  return {k[len(prefix):]: v.to(DT) for k, v in weights.items() if k.startswith(prefix)}


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens, layer_outputs: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
  """logits [T, vocab] of one sequence; `layer_outputs`, when given, receives the sum of the streams after every layer"""
  eps, mult = float(config["norm"]["eps"]), float(config.get("residual_mult", 1.0))
  S = int(config.get("streams", 0))
  has_canon = "canon" in config
  w = {k: v.to(DT) for k, v in weights.items()}
  x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
  x = rms_unit(x, eps) * w["embed.norm"]
  X = [x.clone() for _ in range(max(S, 1))]
  for i, layer in enumerate(config["layers"]):
    p = f"l{i}."
    subs = [(1, lambda h, i=i, layer=layer: mixer(layer["type"], h, sub(weights, f"l{i}.mix."), layer["mixer"], eps))]
    if layer.get("mlp") is not None:
      subs.append((2, lambda h, i=i: feed_forward(h, sub(weights, f"l{i}.mlp."))))
    for qn, fn in subs:
      canon_w = w[p + f"canon{qn}"] if has_canon else None
      if S > 0:
        cin, cout, cmix = w[p + f"hc{qn}.in"], w[p + f"hc{qn}.out"], w[p + f"hc{qn}.mix"]
        u = sum(cin[s] * X[s] for s in range(S))
        y = fn(sublayer_input(u, w[p + f"norm{qn}"], eps, canon_w))
        X = [sum(cmix[s, t] * X[s] for s in range(S)) + mult * cout[t] * y for t in range(S)]
      else:
        y = fn(sublayer_input(X[0], w[p + f"norm{qn}"], eps, canon_w))
        X = [X[0] + mult * y]
    if layer_outputs is not None:
      layer_outputs.append(sum(X))
  x = sum(X)
  x = rms_unit(x, eps) * w["final.norm"]
  return x @ w["head"].T
