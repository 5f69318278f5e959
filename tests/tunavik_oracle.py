"""Plain, slow restatement of the Tunavik design in torch (fp32 or fp64, CPU): one function per mechanism, whole sequences at
once, no cache, no batching.  The product path (the layered-model kernels of libxotb200_lm) shares no code with this file; the
tests compare the two on small random models.

Notation: T tokens, D width, H query heads, G key/value heads, dk query/key size, dv value size per head, B distance buckets,
E experts of inner size F, K experts per token."""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

Tensor = torch.Tensor


# ---- norms, activation, positions --------------------------------------------------------------------------------------------
def rms_unit(x: Tensor, eps: float) -> Tensor:
  """every row divided by sqrt(mean of its squares + eps)"""
  return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_around_zero(x: Tensor, w: Tensor, eps: float) -> Tensor:
  """the block norm: the stored weight is the deviation of the gain from one"""
  return rms_unit(x, eps) * (1.0 + w)


def squared_relu(z: Tensor) -> Tensor:
  r = torch.clamp(z, min=0.0)
  return r * r


def position_vectors(T: int, D: int, dtype) -> Tensor:
  """[T, D]: columns 2i / 2i + 1 hold sin / cos of p * 10000^(-2i / D)"""
  out = torch.zeros(T, D, dtype=dtype)
  p = torch.arange(T, dtype=dtype)
  for i in range((D + 1) // 2):
    a = p * (10000.0 ** (-2.0 * i / D))
    out[:, 2 * i] = torch.sin(a)
    if 2 * i + 1 < D:
      out[:, 2 * i + 1] = torch.cos(a)
  return out


# ---- attention -----------------------------------------------------------------------------------------------------------------
def distance_bucket(n: int, B: int, far: float) -> int:
  """the first B // 2 distances have a bucket each; the rest of the buckets is spread logarithmically up to the distance `far`"""
  h = B // 2
  if n < h:
    return n
  return min(B - 1, h + int(math.floor(math.log(n / h) / math.log(far / h) * (B - h))))


def query_temperature(T: int, coef: float, every: int, dtype) -> Tensor:
  """[T]: the multiplier of the query at position p, 1 + coef * ln(1 + (p + 1) // every)"""
  return torch.tensor([1.0 + coef * math.log((p + 1) // every + 1) for p in range(T)], dtype=dtype)


def attention_keys_values(h: Tensor, W: Dict[str, Tensor], m: dict, eps: float) -> Tuple[Tensor, Tensor]:
  """what an attention layer's cache holds: keys after the norm over the whole key projection [T, G, dk], values [T, G, dv]"""
  T = h.shape[0]
  k = rms_unit(h @ W["k"].T + W["k.b"], eps) * W["k.norm"]
  v = h @ W["v"].T + W["v.b"]
  return k.reshape(T, m["kv_heads"], m["dim"]), v.reshape(T, m["kv_heads"], m["vdim"])


def attention(h: Tensor, W: Dict[str, Tensor], m: dict, eps: float, kv: Optional[Tuple[Tensor, Tensor]] = None) -> Tensor:
  """Causal grouped-query attention without rotation.  Queries (and keys) are normed over the whole projection and the query of
  position p is scaled by its temperature; a learned bias per distance bucket and head is added to the scaled score; the softmax
  runs over the visible keys and one extra logit per head (the sink), which carries no value."""
  T = h.shape[0]
  H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
  q = rms_unit(h @ W["q"].T + W["q.b"], eps) * W["q.norm"]
  t = m.get("q_temp")
  if t:
    q = q * query_temperature(T, t["coef"], t["every"], h.dtype)[:, None]
  q = q.reshape(T, H, dk)
  k, v = kv if kv is not None else attention_keys_values(h, W, m, eps)
  B = W["rel"].shape[0]
  bucket_of = torch.tensor([distance_bucket(n, B, m["bias_max"]) for n in range(T)])
  i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
  bucket = bucket_of[torch.clamp(i - j, min=0)]       # [T, T]; entries above the diagonal are masked below
  out = torch.zeros(T, H, dv, dtype=h.dtype)
  for a in range(H):
    g = a // (H // G)
    s = (q[:, a] @ k[:, g].T) * m["scale"] + W["rel"][:, a][bucket]
    s = s.masked_fill(j > i, float("-inf"))
    z = torch.cat([s, W["sink"][a].expand(T, 1)], dim=1)
    p = torch.softmax(z, dim=1)[:, :T]                # the sink takes its share of the weight and gives nothing back
    out[:, a] = p @ v[:, g]
  return out.reshape(T, H * dv) @ W["o"].T + W["o.b"]


# ---- feed-forward ----------------------------------------------------------------------------------------------------------------
def route(h: Tensor, W: Dict[str, Tensor], r: dict) -> Tuple[Tensor, Tensor]:
  """([T, K] expert ids, [T, K] weights): the K largest logits, softmax over those K only"""
  z = h @ W["router"].T + W["router.b"]
  ids = torch.argsort(z, dim=-1, descending=True, stable=True)[:, : r["top"]]
  return ids, torch.softmax(torch.gather(z, 1, ids), dim=-1)


def route_gap(h: Tensor, W: Dict[str, Tensor], r: dict) -> Tensor:
  """[T]: how far the last chosen logit lies above the best one left out (inf when every expert is chosen): rows where this is
  tiny may legitimately choose otherwise once h is rounded to 16 bits"""
  z = torch.sort(h @ W["router"].T + W["router.b"], dim=-1, descending=True).values
  if r["top"] >= z.shape[1]:
    return torch.full((h.shape[0],), float("inf"), dtype=h.dtype)
  return z[:, r["top"] - 1] - z[:, r["top"]]


def expert(h: Tensor, up: Tensor, down: Tensor) -> Tensor:
  return squared_relu(h @ up.T) @ down.T


def moe_ff(h: Tensor, W: Dict[str, Tensor], mlp: dict) -> Tensor:
  ids, wts = route(h, W, mlp["router"])
  out = torch.zeros_like(h)
  for t in range(h.shape[0]):
    for k in range(ids.shape[1]):
      e = int(ids[t, k])
      out[t] += wts[t, k] * expert(h[t], W[f"e{e}.up"], W[f"e{e}.down"])
  if mlp.get("shared"):
    out = out + expert(h, W["shared.up"], W["shared.down"])
  return out


# ---- the model -------------------------------------------------------------------------------------------------------------------
def sub(weights: Dict[str, Tensor], prefix: str) -> Dict[str, Tensor]:
  return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg: dict, weights: Dict[str, Tensor], tokens, dtype=torch.float64, gaps: Optional[List[Tensor]] = None) -> Tuple[Tensor, List[Tensor]]:
  """(logits [T, vocab], the residual stream after every layer); `gaps` collects every router's route_gap"""
  W = {k: v.to(dtype) for k, v in weights.items()}
  eps, D = cfg["norm"]["eps"], cfg["width"]
  tok = torch.as_tensor(tokens, dtype=torch.long)
  x = norm_around_zero(W["embed"][tok] + position_vectors(len(tok), D, dtype), W["embed.norm"], eps)
  held: Dict[int, Tuple[Tensor, Tensor]] = {}
  trail = []
  for i, layer in enumerate(cfg["layers"]):
    m, Wm = layer["mixer"], sub(W, f"l{i}.mix.")
    src = m.get("kv_from")
    if src is None:
      held[i] = attention_keys_values(x, Wm, m, eps)
    x = x + norm_around_zero(attention(x, Wm, m, eps, held[i if src is None else src]), W[f"l{i}.norm1"], eps)
    if layer.get("mlp") is not None:
      if gaps is not None:
        gaps.append(route_gap(x, sub(W, f"l{i}.mlp."), layer["mlp"]["router"]))
      x = x + norm_around_zero(moe_ff(x, sub(W, f"l{i}.mlp."), layer["mlp"]), W[f"l{i}.norm2"], eps)
    trail.append(x)
  lg = (norm_around_zero(x, W["final.norm"], eps) @ W["head"].T) * cfg.get("logit_scale", 1.0)
  cap = cfg.get("logit_softcap")
  if cap:
    lg = cap * torch.tanh(lg / cap)
  return lg, trail


def tensor_shapes(cfg: dict, buckets=16) -> Dict[str, Tuple[int, ...]]:
  """names and shapes of a model's tensors; `buckets`: rows of the distance-bias tables (one number, or one per layer)"""
  D, V = cfg["width"], cfg["vocab"]
  out = {"embed": (V, D), "embed.norm": (D,), "final.norm": (D,), "head": (V, D)}
  for i, layer in enumerate(cfg["layers"]):
    p, m = f"l{i}.", layer["mixer"]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    out[p + "norm1"] = (D,)
    out[p + "mix.q"], out[p + "mix.q.b"], out[p + "mix.q.norm"] = (H * dk, D), (H * dk,), (H * dk,)
    if m.get("kv_from") is None:
      out[p + "mix.k"], out[p + "mix.k.b"], out[p + "mix.k.norm"] = (G * dk, D), (G * dk,), (G * dk,)
      out[p + "mix.v"], out[p + "mix.v.b"] = (G * dv, D), (G * dv,)
    out[p + "mix.rel"], out[p + "mix.sink"] = (buckets if isinstance(buckets, int) else buckets[i], H), (H,)
    out[p + "mix.o"], out[p + "mix.o.b"] = (D, H * dv), (D,)
    mlp = layer.get("mlp")
    if mlp is not None:
      out[p + "norm2"] = (D,)
      E, F = mlp["router"]["experts"], mlp["expert"]["ff"]
      out[p + "mlp.router"], out[p + "mlp.router.b"] = (E, D), (E,)
      for e in range(E):
        out[p + f"mlp.e{e}.up"], out[p + f"mlp.e{e}.down"] = (F, D), (D, F)
      if mlp.get("shared"):
        out[p + "mlp.shared.up"], out[p + "mlp.shared.down"] = (mlp["shared"]["ff"], D), (D, mlp["shared"]["ff"])
  return out


def random_weights(cfg: dict, seed: int, buckets=16) -> Dict[str, Tensor]:
  """bf16-representable random weights (so a 16-bit engine and this oracle start from identical numbers)"""
  g = torch.Generator().manual_seed(seed)
  out = {}
  for name, shape in tensor_shapes(cfg, buckets).items():
    if name.endswith("router"):
      t = 3.0 * torch.randn(shape, generator=g) / math.sqrt(shape[1])     # spread logits: no near-ties between experts
    elif name.endswith(".rel"):
      t = 1.5 * torch.randn(shape, generator=g)       # a bias one bucket off moves the weights visibly
    elif name.endswith(".sink"):
      t = 1.0 + torch.randn(shape, generator=g)       # sinks that take a real share of the weight
    elif name.endswith(("q.norm", "k.norm")):
      t = 1.0 + 0.2 * torch.randn(shape, generator=g)
    elif len(shape) == 1:
      t = 0.3 * torch.randn(shape, generator=g)       # block norms (stored around zero) and biases
    elif name == "embed":
      t = torch.randn(shape, generator=g)
    else:
      t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
    out[name] = t.to(torch.bfloat16).to(torch.float32)
  return out
