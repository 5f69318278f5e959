"""`LayeredShard` — synchronous Python owner of one `xotb200_lm*` (include/xotb200_lm.h): models given as a list of layers whose
token mixers differ (latent attention, attention over a key/value cache, delta-rule recurrences) and keep different per-request state.  It offers the methods the
rest of the package uses on `NativeShard` (`load_dir / begin_request / begin_batch / select_request / clear_request / forward /
last_token / close / kernel_launches / weight_bytes`) plus the batched `step`, so `B200ShardInferenceEngine`, the Cheetah
service and the schedulers drive it unchanged.  All compute is in libxotb200_lm.so; there is no CPU fallback.

A model family is a function config.json -> list of `LayerSpec` (see `zokuvik_layers`, `bufulorn_layers`): the library knows
mechanisms and their parameters, not families."""
from __future__ import annotations

import ctypes as C
import json
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import _lib
from ._lib import LmCfg, LmLayer, check_lm

DEFAULT_PAGE = 64


@dataclass
class LayerSpec:
  """one layer of a layered model; the fields are those of xotb200_lm_layer"""
  mixer: int
  heads: int
  dim: int
  vdim: int = 0
  rot_dim: int = 0
  kv_rank: int = 0
  q_rank: int = 0
  rot_dims: int = 0
  rot_layout: int = _lib.LM_ROT_INTERLEAVED
  window: int = 0
  out_gate: int = 0
  low_rank: int = 0
  ff: int = 0
  rot_base: float = 10000.0
  scale: float = 1.0
  kv_heads: int = 0
  kv_from: int = -1
  chunk: int = 0
  qk_norm: int = 0
  proj_bias: int = 0
  dist_bias: int = 0
  conv_taps: int = 0
  ff_kind: int = _lib.LM_FF_RELU2
  experts: int = 0
  expert_ff: int = 0
  top: int = 0
  groups: int = 0
  groups_keep: int = 0
  softcap: float = 0.0
  out_bias: int = 0
  sink: int = 0
  rel_buckets: int = 0
  rel_max: float = 0.0
  q_temp_coef: float = 0.0
  q_temp_every: int = 0
  expert_act: int = _lib.LM_EXPERT_SILU_GATED
  router_kind: int = _lib.LM_ROUTER_SOFTMAX_ALL
  router_bias: int = 0
  shared_ff: int = 0
  rot_scale_factor: float = 0.0
  rot_scale_low: float = 0.0
  rot_scale_high: float = 0.0
  rot_scale_original: float = 0.0
  keep_first: int = 0
  pool: int = 0
  gate_cap: float = 0.0
  out_norm_groups: int = 0
  par_on: int = 0
  par_mixer: int = 0
  par_heads: int = 0
  par_kv_heads: int = 0
  par_dim: int = 0
  par_vdim: int = 0
  par_conv_taps: int = 0
  par_out_norm_groups: int = 0
  par_gate_cap: float = 0.0
  mix_scale: float = 1.0
  par_scale: float = 0.0

  def to_c(self) -> LmLayer:
    c = LmLayer()
    for name, _ in LmLayer._fields_:
      setattr(c, name, getattr(self, name))
    return c


def read_tensor_shapes(model_dir) -> Dict[str, Tuple[int, ...]]:
  """name -> shape from the headers of every *.safetensors in the directory (8-byte little-endian length + JSON)"""
  shapes: Dict[str, Tuple[int, ...]] = {}
  files = sorted(Path(model_dir).glob("*.safetensors"))
  if not files:
    raise FileNotFoundError(f"no *.safetensors in {model_dir}")
  for f in files:
    with open(f, "rb") as fh:
      n = struct.unpack("<Q", fh.read(8))[0]
      hdr = json.loads(fh.read(n))
    for k, v in hdr.items():
      if k != "__metadata__":
        shapes[k] = tuple(int(x) for x in v["shape"])
  return shapes


# ---- the Zokuvik family ------------------------------------------------------------------------------------------------------
# config.json: {"architecture": "Zokuvik", "width", "vocab", "norm": {"eps", "groups"}, "layers": [{"type", "mixer": {...}, "mlp"}]}
#   type "latent_attention"    queries through a normed latent, pairs (2i, 2i+1) rotated, causal, one output gate per head
#   type "latent_attention_2"  direct queries, pairs (i, i + dims/2) rotated, sliding window mixer.mask.size, no gate
#   type "general_delta"       delta-rule recurrence; the inner size of its decay branch is the first dimension of l<i>.mix.w1
ZOKUVIK_ATTENTION = {
  "latent_attention": dict(q_latent=True, rot_layout=_lib.LM_ROT_INTERLEAVED, out_gate=1),
  "latent_attention_2": dict(q_latent=False, rot_layout=_lib.LM_ROT_HALF, out_gate=0),
}


def zokuvik_layers(config: dict, shapes: Dict[str, Tuple[int, ...]]) -> List[LayerSpec]:
  out = []
  for i, layer in enumerate(config["layers"]):
    kind, m, mlp = layer["type"], layer["mixer"], layer.get("mlp")
    if mlp is not None and mlp.get("kind", "dense") != "dense":
      raise ValueError(f"layer {i}: feed-forward kind {mlp.get('kind')!r} is not implemented (dense only)")
    ff = int(mlp["ff"]) if mlp is not None else 0
    if kind in ZOKUVIK_ATTENTION:
      opt = ZOKUVIK_ATTENTION[kind]
      rot = m.get("rot") or {}
      mask = m.get("mask") or {}
      out.append(LayerSpec(
        mixer=_lib.LM_MIX_LATENT_ATTN, heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]), rot_dim=int(m["rot_dim"]),
        kv_rank=int(m["kv_rank"]), q_rank=int(m["q_rank"]) if opt["q_latent"] else 0,
        rot_dims=int(rot.get("dims", m["rot_dim"])), rot_layout=opt["rot_layout"], rot_base=float(rot.get("base", 10000.0)),
        window=int(mask.get("size", 0)), out_gate=opt["out_gate"], scale=float(m["scale"]), ff=ff))
    elif kind == "general_delta":
      w1 = shapes.get(f"l{i}.mix.w1")
      if w1 is None:
        raise ValueError(f"layer {i}: tensor l{i}.mix.w1 (which gives the decay branch its inner size) is missing")
      out.append(LayerSpec(mixer=_lib.LM_MIX_DELTA_RULE, heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["dim"]),
                           low_rank=int(w1[0]), ff=ff))
    else:
      raise ValueError(f"layer {i}: mixer type {kind!r} is not implemented")
  return out


def zokuvik_globals(config: dict) -> dict:
  return dict(width=int(config["width"]), vocab=int(config["vocab"]), norm_groups=int(config["norm"]["groups"]),
              norm_eps=float(config["norm"]["eps"]))


# ---- the Bufulorn family -----------------------------------------------------------------------------------------------------
# config.json: {"architecture": "Bufulorn", "width", "vocab", "max_positions", "norm": {"eps"}, "layers": [{"type", "mixer", "mlp"}]}
# A layer is x += LN(mixer(x)), x += LN(ff(x)) (layer norms with weight and bias on the sublayers' outputs); a learned position
# vector is added to the embedding.
#   type "attention"  grouped-query attention (mixer: heads, kv_heads, dim, vdim, scale, softcap, mask.size = block of the
#                     block-local causal mask, kv_from = layer whose keys/values it reads): biased projections, per-head RMS norm of
#                     queries and keys, logarithmic distance penalty, no rotation, one sigmoid gate per output entry
#   type "delta"      gated delta rule (mixer: heads, kv_heads, dim, vdim, conv = taps of the short convolutions)
#   mlp.kind "dense"  W_down xIELU(W_up h) (mlp.ff);  "moe": mlp.router {experts, top, groups {count, keep}}, mlp.expert.ff
def _bufulorn_ff(i: int, mlp) -> dict:
  if mlp is None:
    return dict(ff=0, ff_kind=_lib.LM_FF_XIELU)
  kind = mlp.get("kind", "dense")
  if kind == "dense":
    return dict(ff=int(mlp["ff"]), ff_kind=_lib.LM_FF_XIELU)
  if kind == "moe":
    r = mlp["router"]
    groups = r.get("groups") or {}
    return dict(ff=0, ff_kind=_lib.LM_FF_MOE, experts=int(r["experts"]), top=int(r["top"]), expert_ff=int(mlp["expert"]["ff"]),
                groups=int(groups.get("count", 0)), groups_keep=int(groups.get("keep", groups.get("count", 0))))
  raise ValueError(f"layer {i}: feed-forward kind {kind!r} is not implemented (dense, moe)")


def bufulorn_layers(config: dict, shapes: Dict[str, Tuple[int, ...]]) -> List[LayerSpec]:
  out = []
  for i, layer in enumerate(config["layers"]):
    kind, m = layer["type"], layer["mixer"]
    ff = _bufulorn_ff(i, layer.get("mlp"))
    if kind == "attention":
      src = m.get("kv_from")
      out.append(LayerSpec(
        mixer=_lib.LM_MIX_ATTENTION, heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]), vdim=int(m["vdim"]),
        scale=float(m["scale"]), softcap=float(m.get("softcap") or 0.0), chunk=int((m.get("mask") or {}).get("size", 0)),
        kv_from=-1 if src is None else int(src), qk_norm=1, proj_bias=1, dist_bias=1, out_gate=2, **ff))
    elif kind == "delta":
      out.append(LayerSpec(mixer=_lib.LM_MIX_GATED_DELTA, heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
                           vdim=int(m["vdim"]), conv_taps=int(m["conv"]), **ff))
    else:
      raise ValueError(f"layer {i}: mixer type {kind!r} is not implemented")
  return out


def bufulorn_globals(config: dict) -> dict:
  return dict(width=int(config["width"]), vocab=int(config["vocab"]), norm_groups=1, norm_eps=float(config["norm"]["eps"]),
              block=_lib.LM_BLOCK_POST_LN, max_positions=int(config["max_positions"]))


# ---- the Tunavik family ------------------------------------------------------------------------------------------------------
# config.json: {"architecture": "Tunavik", "width", "vocab", "norm": {"eps"}, "logit_scale", "logit_softcap", "layers": [{"type", "mixer", "mlp"}]}
# A layer is x += rms(mixer(x)) * (1 + w), x += rms(ff(x)) * (1 + w); a sine/cosine position vector (base 10000) is added to the
# embedding and the sum is normed the same way (embed.norm); the logits are scaled and soft-capped.
#   type "attention"  grouped-query attention (mixer: heads, kv_heads, dim, vdim, scale, bias_max, q_temp {coef, every}, kv_from):
#                     biased q / k / v / o projections, ONE RMS norm over the whole query (key) projection, no rotation, query
#                     temperature by position, learned bias per logarithmic distance bucket (table l<i>.mix.rel, whose first
#                     dimension is the number of buckets), one sink logit per head in the softmax denominator
#   mlp.kind "moe"    relu^2 experts without biases (mlp.expert.ff), router with bias: the `top` largest logits, softmax over them
#                     (mlp.router {experts, top}); optional shared expert of the same form (mlp.shared.ff)
TUNAVIK_SINUSOID_BASE = 10000.0


def _tunavik_ff(i: int, mlp) -> dict:
  if mlp is None:
    return dict(ff=0, ff_kind=_lib.LM_FF_MOE, experts=0)
  kind = mlp.get("kind")
  if kind != "moe":
    raise ValueError(f"layer {i}: feed-forward kind {kind!r} is not implemented (moe)")
  r = mlp["router"]
  shared = mlp.get("shared") or {}
  return dict(ff=0, ff_kind=_lib.LM_FF_MOE, experts=int(r["experts"]), top=int(r["top"]), expert_ff=int(mlp["expert"]["ff"]),
              expert_act=_lib.LM_EXPERT_RELU2, router_kind=_lib.LM_ROUTER_TOPK_SOFTMAX, router_bias=1, shared_ff=int(shared.get("ff", 0)))


def tunavik_layers(config: dict, shapes: Dict[str, Tuple[int, ...]]) -> List[LayerSpec]:
  out = []
  for i, layer in enumerate(config["layers"]):
    kind, m = layer["type"], layer["mixer"]
    if kind != "attention":
      raise ValueError(f"layer {i}: mixer type {kind!r} is not implemented")
    rel = shapes.get(f"l{i}.mix.rel")
    if rel is None or len(rel) != 2:
      raise ValueError(f"layer {i}: tensor l{i}.mix.rel (whose first dimension is the number of distance buckets) is missing")
    temp = m.get("q_temp") or {}
    src = m.get("kv_from")
    out.append(LayerSpec(
      mixer=_lib.LM_MIX_ATTENTION, heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]), vdim=int(m["vdim"]),
      scale=float(m["scale"]), kv_from=-1 if src is None else int(src), qk_norm=_lib.LM_QKNORM_ROW, proj_bias=1, out_bias=1, sink=1,
      rel_buckets=int(rel[0]), rel_max=float(m["bias_max"]), q_temp_coef=float(temp.get("coef", 0.0)), q_temp_every=int(temp.get("every", 1)),
      **_tunavik_ff(i, layer.get("mlp"))))
  return out


def tunavik_globals(config: dict) -> dict:
  return dict(width=int(config["width"]), vocab=int(config["vocab"]), norm_groups=1, norm_eps=float(config["norm"]["eps"]),
              block=_lib.LM_BLOCK_POST_RMS, pos_sinusoid=1, sinusoid_base=TUNAVIK_SINUSOID_BASE, embed_norm=1,
              logit_scale=float(config.get("logit_scale", 1.0)), logit_softcap=float(config.get("logit_softcap") or 0.0))


# ---- the Fubelorn family -----------------------------------------------------------------------------------------------------
# config.json: {"architecture": "Fubelorn", "width", "vocab", "norm": {"eps"}, "residual_mult", "streams", "canon": {"taps"},
#               "layers": [{"type", "mixer", "mlp"}]}
# A layer is pre-norm with ONE-NUMBER norm weights: x += mult * sublayer(c(rms(x) * g)), c(h) = h + causal convolution of h over
# time (canon.taps); the stream is kept in `streams` copies mixed by hyper-connections (l<i>.hc<q>.in / out / mix); embedding and
# final norm are of the same kind.  Mixers:
#   type "parallel"    left: attention without rotation, weightless RMS norm of every query / key head, sliding window mask.size that
#                      keeps the first mask.keep_first tokens;  right: gated delta rule (heads, kv_heads, dim, vdim, conv)
#   type "parallel_2"  left: rotary attention (rot {base, dims, scaling {factor, low, high, original}}, pairs (i, i + dims / 2)), sliding
#                      window mask.size with pooled blocks of mask.pool tokens beyond it, one sigmoid gate per head;
#                      right: matrix LSTM (heads, dim, vdim, gate_cap)
#   type "mamba2"      state-space layer (heads, vdim, state, groups, norm_groups, conv)
#   output of a two-mixer layer: left_scale * left + right_scale * right.        mlp.kind "dense": W_down gelu(W_up h) (mlp.ff)
# Which options a left mixer has follows from its keys (rot, mask.keep_first, mask.pool) and from the layer type (query/key norm
# for "parallel", head gate for "parallel_2").
FUBELORN_LEFT = {"parallel": dict(qk_norm=_lib.LM_QKNORM_HEAD_PLAIN, out_gate=0), "parallel_2": dict(qk_norm=_lib.LM_QKNORM_NONE, out_gate=1)}


def _fubelorn_attention(i: int, kind: str, m: dict) -> dict:
  mask, rot = m.get("mask") or {}, m.get("rot") or None
  out = dict(mixer=_lib.LM_MIX_ATTENTION, heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]), vdim=int(m["vdim"]),
             scale=float(m["scale"]), window=int(mask.get("size", 0)), keep_first=int(mask.get("keep_first", 0)), pool=int(mask.get("pool", 0)),
             **FUBELORN_LEFT[kind])
  if out["window"] == 0:                                # no window: every earlier token is seen as itself, nothing to keep or pool
    out.update(keep_first=0, pool=0)
  if rot:
    out.update(rot_dims=int(rot["dims"]), rot_base=float(rot["base"]), rot_layout=_lib.LM_ROT_HALF)
    sc = rot.get("scaling")
    if sc:
      out.update(rot_scale_factor=float(sc["factor"]), rot_scale_low=float(sc["low"]), rot_scale_high=float(sc["high"]), rot_scale_original=float(sc["original"]))
  return out


def _fubelorn_recurrent(i: int, kind: str, m: dict) -> dict:
  """fields of a recurrent mixer under the names of a layer's FIRST mixer"""
  if kind == "parallel":
    return dict(mixer=_lib.LM_MIX_GATED_DELTA, heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]), vdim=int(m["vdim"]),
                conv_taps=int(m["conv"]))
  if kind == "parallel_2":
    return dict(mixer=_lib.LM_MIX_MATRIX_LSTM, heads=int(m["heads"]), kv_heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]), gate_cap=float(m["gate_cap"]))
  return dict(mixer=_lib.LM_MIX_MAMBA2, heads=int(m["heads"]), kv_heads=int(m.get("groups", 1)), dim=int(m["state"]), vdim=int(m["vdim"]),
              conv_taps=int(m["conv"]), out_norm_groups=int(m.get("norm_groups", 1)))


def fubelorn_layers(config: dict, shapes: Dict[str, Tuple[int, ...]]) -> List[LayerSpec]:
  out = []
  for i, layer in enumerate(config["layers"]):
    kind, m, mlp = layer["type"], layer["mixer"], layer.get("mlp")
    if mlp is not None and mlp.get("kind", "dense") != "dense":
      raise ValueError(f"layer {i}: feed-forward kind {mlp.get('kind')!r} is not implemented (dense)")
    ff = dict(ff=int(mlp["ff"]) if mlp is not None else 0, ff_kind=_lib.LM_FF_GELU)
    if kind in FUBELORN_LEFT:
      right = _fubelorn_recurrent(i, kind, m["right"])
      par = dict(par_on=1, par_mixer=right["mixer"], par_heads=right["heads"], par_kv_heads=right["kv_heads"], par_dim=right["dim"], par_vdim=right["vdim"],
                 par_conv_taps=right.get("conv_taps", 0), par_out_norm_groups=right.get("out_norm_groups", 0), par_gate_cap=right.get("gate_cap", 0.0),
                 mix_scale=float(m.get("left_scale", 1.0)), par_scale=float(m.get("right_scale", 1.0)))
      out.append(LayerSpec(**_fubelorn_attention(i, kind, m["left"]), **par, **ff))
    elif kind == "mamba2":
      out.append(LayerSpec(**_fubelorn_recurrent(i, kind, m), **ff))
    else:
      raise ValueError(f"layer {i}: mixer type {kind!r} is not implemented")
  return out


def fubelorn_globals(config: dict) -> dict:
  return dict(width=int(config["width"]), vocab=int(config["vocab"]), norm_groups=1, norm_eps=float(config["norm"]["eps"]),
              block=_lib.LM_BLOCK_PRE_SCALAR, embed_norm=1, streams=int(config.get("streams", 0)),
              canon_taps=int((config.get("canon") or {}).get("taps", 0)), residual_mult=float(config.get("residual_mult", 1.0)))


LAYERED_FAMILIES = {"Zokuvik": (zokuvik_layers, zokuvik_globals), "Bufulorn": (bufulorn_layers, bufulorn_globals),
                    "Tunavik": (tunavik_layers, tunavik_globals), "Fubelorn": (fubelorn_layers, fubelorn_globals)}


class LayeredShard:
  def __init__(self, config: dict, device: int = 0, dtype: str = "bfloat16"):
    fam = config.get("architecture")
    if fam not in LAYERED_FAMILIES:
      raise ValueError(f"architecture {fam!r} is not a layered model family known here ({sorted(LAYERED_FAMILIES)})")
    if dtype not in ("bfloat16", "float32"):
      raise ValueError(f"dtype {dtype!r}: the layered engine serves in bfloat16 and has an all-float32 mode")
    self.lib = _lib.load_lm()
    self.config, self.family, self.device, self.dtype = dict(config), fam, int(device), dtype
    self.globals = LAYERED_FAMILIES[fam][1](config)
    self.n_layers = len(config["layers"])
    self.h = None
    self.start = self.end = -1
    self.cur = 0                      # slot that forward() acts on (select_request)
    self.n_slots = 0
    self._last_token = None

  # -- lifetime / weights -------------------------------------------------------------------------------------------------
  def close(self):
    if getattr(self, "h", None):
      self.lib.xotb200_lm_destroy(self.h)
      self.h = None

  def __del__(self):
    try:
      self.close()
    except Exception:
      pass

  @property
  def is_first(self) -> bool: return self.start == 0
  @property
  def is_last(self) -> bool: return self.end == self.n_layers - 1
  @property
  def vocab(self) -> int: return self.globals["vocab"]
  @property
  def width(self) -> int: return self.globals["width"]
  @property
  def max_positions(self) -> int:
    """most tokens a request may hold (a learned position table ends there); 0 = no such limit"""
    return int(self.globals.get("max_positions", 0))

  def set_shard(self, start_layer: int, end_layer: int, shapes: Dict[str, Tuple[int, ...]]):
    """create the native engine for layers [start_layer, end_layer]; `shapes` = tensor name -> shape (sizes that only a
    tensor's shape gives are read from it)"""
    self.close()
    specs = LAYERED_FAMILIES[self.family][0](self.config, shapes)
    cfg = LmCfg()
    cfg.n_layers, cfg.start_layer, cfg.end_layer = self.n_layers, int(start_layer), int(end_layer)
    cfg.width, cfg.vocab, cfg.norm_groups = self.globals["width"], self.globals["vocab"], self.globals["norm_groups"]
    cfg.norm_eps = self.globals["norm_eps"]
    cfg.block, cfg.max_positions = self.globals.get("block", _lib.LM_BLOCK_GROUP_RMS), self.globals.get("max_positions", 0)
    cfg.pos_sinusoid, cfg.sinusoid_base = self.globals.get("pos_sinusoid", 0), self.globals.get("sinusoid_base", 0.0)
    cfg.embed_norm = self.globals.get("embed_norm", 0)
    cfg.logit_scale, cfg.logit_softcap = self.globals.get("logit_scale", 1.0), self.globals.get("logit_softcap", 0.0)
    cfg.streams, cfg.canon_taps = self.globals.get("streams", 0), self.globals.get("canon_taps", 0)
    cfg.residual_mult = self.globals.get("residual_mult", 0.0)
    cfg.dtype = _lib.LM_DTYPE_F32 if self.dtype == "float32" else _lib.LM_DTYPE_BF16
    arr = (LmLayer * len(specs))(*[s.to_c() for s in specs])
    h = C.c_void_p()
    check_lm(self.lib.xotb200_lm_create(C.byref(cfg), arr, self.device, C.byref(h)))
    self.h, self.specs = h, specs
    self.start, self.end = int(start_layer), int(end_layer)
    self.n_slots = 0

  def load_dir(self, model_dir, start_layer: int = 0, end_layer: Optional[int] = None):
    end_layer = self.n_layers - 1 if end_layer is None else end_layer
    self.set_shard(start_layer, end_layer, read_tensor_shapes(model_dir))
    check_lm(self.lib.xotb200_lm_load_dir(self.h, str(model_dir).encode()))

  def load_tensor(self, name: str, bf16_bits: np.ndarray) -> bool:
    a = np.ascontiguousarray(bf16_bits)
    assert a.dtype in (np.uint16, np.int16), "pass bf16 bit patterns (uint16)"
    shp = (C.c_int64 * a.ndim)(*a.shape)
    return check_lm(self.lib.xotb200_lm_load_tensor(self.h, name.encode(), a.ctypes.data_as(C.c_void_p), shp, a.ndim)) == 0

  def init_synthetic(self, seed: int = 1234):
    """random weights made on the device (after set_shard): benchmarks and smoke runs"""
    check_lm(self.lib.xotb200_lm_init_synthetic(self.h, int(seed)))

  def check_loaded(self):
    check_lm(self.lib.xotb200_lm_check_loaded(self.h))

  # -- request state --------------------------------------------------------------------------------------------------------
  def begin_pool(self, max_tokens: int, max_requests: int, page_size: int = DEFAULT_PAGE):
    """cache for at most max_requests live requests holding at most max_tokens tokens together"""
    check_lm(self.lib.xotb200_lm_begin(self.h, int(max_tokens), int(max_requests), int(page_size)))
    self.n_slots, self.cur = int(max_requests), 0

  def begin_request(self, max_total_len: int):
    self.begin_pool(max_total_len, 1)

  def begin_batch(self, max_total_len: int, n_requests: int):
    """n_requests slots of up to max_total_len tokens each (the shard engine's call: one KV cache per request)"""
    self.begin_pool(int(max_total_len) * int(n_requests), n_requests)

  def select_request(self, request: int):
    if not 0 <= int(request) < self.n_slots:
      raise ValueError(f"request slot {request} out of range ({self.n_slots})")
    self.cur = int(request)

  def clear_request(self, request: int):
    check_lm(self.lib.xotb200_lm_clear_request(self.h, int(request)))

  def request_len(self, request: int) -> int:
    v = C.c_int()
    check_lm(self.lib.xotb200_lm_request_len(self.h, int(request), C.byref(v)))
    return int(v.value)

  # -- the step ---------------------------------------------------------------------------------------------------------------
  def step(self, slots: Sequence[int], rows: Sequence[np.ndarray], want: Optional[Sequence[int]] = None, logits: bool = True,
           argmax: bool = True):
    """One batched step.  rows[i]: the next token ids (1-D int) of slot slots[i] on the first shard, else its hidden state
    [n_i, width] float32.  want: packed row indices whose output is asked for (default: every request's last row).
    Last shard -> (logits [n_want, vocab] float32 | None, argmax [n_want] int32 | None); other shards -> hidden [sum n_i, width]."""
    n_seq = len(slots)
    if self.is_first:
      parts = [np.ascontiguousarray(r, dtype=np.int32).reshape(-1) for r in rows]
      counts = np.array([p.size for p in parts], dtype=np.int32)
      tok = np.ascontiguousarray(np.concatenate(parts)) if parts else np.zeros(0, np.int32)
      tok_p, hid_p = tok.ctypes.data_as(C.c_void_p), None
    else:
      parts = [np.ascontiguousarray(r, dtype=np.float32).reshape(-1, self.width) for r in rows]
      counts = np.array([p.shape[0] for p in parts], dtype=np.int32)
      hid = np.ascontiguousarray(np.concatenate(parts, axis=0))
      tok_p, hid_p = None, hid.ctypes.data_as(C.c_void_p)
    M = int(counts.sum())
    sl = np.ascontiguousarray(slots, dtype=np.int32)
    if want is None:
      want = (np.cumsum(counts) - 1)
    wn = np.ascontiguousarray(want, dtype=np.int32).reshape(-1)
    lg = am = ho = None
    if self.is_last:
      lg = np.empty((wn.size, self.vocab), dtype=np.float32) if logits else None
      am = np.empty(wn.size, dtype=np.int32) if argmax else None
    else:
      ho = np.empty((M, self.width), dtype=np.float32)
    p = lambda a: a.ctypes.data_as(C.c_void_p) if a is not None else None
    check_lm(self.lib.xotb200_lm_step(self.h, n_seq, p(sl), p(counts), tok_p, hid_p, p(wn), int(wn.size) if self.is_last else 0, p(lg), p(am), p(ho)))
    if self.is_last:
      return lg, am
    return ho

  def forward(self, input_data: np.ndarray, pos0: int) -> np.ndarray:
    """The single-request step of the engine protocol on the selected slot: ndim 2 int ids [1, S] (first shard) or ndim 3
    float32 hidden [1, S, D] -> hidden [1, S, D] float32, or the last position's logits [1, V] on the last shard.  pos0 == 0
    starts the request anew (the slot is emptied); otherwise pos0 must be the slot's length: a recurrent state cannot rewind."""
    a = np.asarray(input_data)
    if a.ndim not in (2, 3):
      raise ValueError(f"input_data.ndim must be 2 (token ids) or 3 (hidden state), got {a.ndim}")
    have = self.request_len(self.cur)
    if pos0 == 0 and have:
      self.clear_request(self.cur)
    elif pos0 != 0 and pos0 != have:
      raise ValueError(f"slot {self.cur} holds {have} tokens; a step at position {pos0} would skip or rewind its state")
    out = self.step([self.cur], [a[0]])
    if self.is_last:
      self._last_token = int(out[1][0])
      return out[0].reshape(1, -1)
    return out.reshape(1, -1, self.width)

  def last_token(self) -> int:
    if self._last_token is None:
      raise RuntimeError("no last-shard step has run yet")
    return self._last_token

  # -- introspection ----------------------------------------------------------------------------------------------------------
  def set_trace(self, on: bool):
    check_lm(self.lib.xotb200_lm_set_trace(self.h, 1 if on else 0))

  def read_trace(self, rows: int) -> np.ndarray:
    """[local layers, rows, width]: the residual stream after every layer of the most recent step"""
    out = np.empty((self.end - self.start + 1, rows, self.width), dtype=np.float32)
    check_lm(self.lib.xotb200_lm_read_trace(self.h, out.ctypes.data_as(C.c_void_p), out.size))
    return out

  def set_gemm_mode(self, mode: int):
    check_lm(self.lib.xotb200_lm_set_gemm_mode(self.h, int(mode)))

  def kernel_launches(self) -> int:
    v = C.c_int64()
    check_lm(self.lib.xotb200_lm_kernel_launches(self.h, C.byref(v)))
    return int(v.value)

  def set_graphs(self, on: bool):
    check_lm(self.lib.xotb200_lm_set_graphs(self.h, 1 if on else 0))

  def graph_replays(self) -> int:
    v = C.c_int64()
    check_lm(self.lib.xotb200_lm_graph_replays(self.h, C.byref(v)))
    return int(v.value)

  def set_attention_mode(self, mode: int):
    check_lm(self.lib.xotb200_lm_set_attention_mode(self.h, int(mode)))

  def prompt_attention_launches(self) -> int:
    v = C.c_int64()
    check_lm(self.lib.xotb200_lm_prompt_attention_launches(self.h, C.byref(v)))
    return int(v.value)

  def tensor_core_launches(self) -> int:
    v = C.c_int64()
    check_lm(self.lib.xotb200_lm_tensor_core_launches(self.h, C.byref(v)))
    return int(v.value)

  def weight_bytes(self) -> int:
    v = C.c_int64()
    check_lm(self.lib.xotb200_lm_weight_bytes(self.h, C.byref(v)))
    return int(v.value)

  def cache_stats(self) -> dict:
    t, f, p = C.c_int(), C.c_int(), C.c_int()
    check_lm(self.lib.xotb200_lm_cache_stats(self.h, C.byref(t), C.byref(f), C.byref(p)))
    return {"pages_total": int(t.value), "pages_free": int(f.value), "page_size": int(p.value)}

  def last_step_ms(self) -> float:
    v = C.c_float()
    check_lm(self.lib.xotb200_lm_last_step_ms(self.h, C.byref(v)))
    return float(v.value)


class RequestSlots:
  """request id -> slot of a `LayeredShard`'s request table.  A request takes the lowest free slot at its first step and keeps it
  until it is released; releasing returns the slot's cache pages to the pool and zeroes its recurrent states, so the next
  owner starts clean.  The batch scheduler and the trace replayer share this table."""

  def __init__(self, native: LayeredShard):
    if native.n_slots < 1:
      raise ValueError("the engine has no request state yet (begin_pool / begin_batch first)")
    self.native = native
    self.by_id: Dict[str, int] = {}
    self.free: List[int] = list(range(native.n_slots))

  def __contains__(self, request_id: str) -> bool:
    return request_id in self.by_id

  def __len__(self) -> int:
    return len(self.by_id)

  def acquire(self, request_id: str) -> int:
    """the request's slot; a request seen for the first time gets a free one"""
    slot = self.by_id.get(request_id)
    if slot is None:
      if not self.free:
        raise RuntimeError(f"all {self.native.n_slots} request slots are taken; request {request_id!r} has to wait")
      slot = self.free.pop(0)
      self.by_id[request_id] = slot
    return slot

  def release(self, request_id: str) -> None:
    slot = self.by_id.pop(request_id, None)
    if slot is not None:
      self.native.clear_request(slot)
      self.free.append(slot)
      self.free.sort()
