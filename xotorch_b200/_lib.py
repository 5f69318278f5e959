"""ctypes binding of libxotb200.so (include/xotb200.h).  This is the stub a maintainer of the reference would add
(see INTEGRATION.md).  There is NO fallback: if the CUDA library is missing or fails to load, importing the
engine raises — the product path never runs on the CPU or through oracle/."""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libxotb200.so"

IPC_HANDLE_BYTES = 64
DTYPE_BF16, DTYPE_F16 = 0, 1
ROPE_PLAIN, ROPE_LLAMA3 = 0, 1
E_TIMEOUT = -5


class ModelCfg(C.Structure):
  """xotb200_model_cfg — mirror of the dict built by load_model_config
  (/root/reference/xotorch/inference/llm_utils.py:79-126)."""
  _fields_ = [
    ("n_layers", C.c_int32), ("dim", C.c_int32), ("ffn", C.c_int32), ("n_heads", C.c_int32),
    ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("vocab", C.c_int32), ("max_pos", C.c_int32),
    ("rope_theta", C.c_float), ("norm_eps", C.c_float), ("tie_embeddings", C.c_int32), ("dtype", C.c_int32),
    ("rope_kind", C.c_int32), ("rope_factor", C.c_float), ("rope_low_freq_factor", C.c_float),
    ("rope_high_freq_factor", C.c_float), ("rope_old_context_len", C.c_int32),
    ("n_experts", C.c_int32), ("experts_per_tok", C.c_int32),
  ]


class XotB200Error(RuntimeError):
  def __init__(self, code: int, msg: str):
    super().__init__(f"xotb200 error {code}: {msg}")
    self.code = code


_lib = None

_SIGS = {
  "xotb200_last_error": (C.c_char_p, []),
  "xotb200_version": (C.c_char_p, []),
  "xotb200_create": (C.c_int, [C.POINTER(ModelCfg), C.c_int, C.POINTER(C.c_void_p)]),
  "xotb200_destroy": (C.c_int, [C.c_void_p]),
  "xotb200_set_shard": (C.c_int, [C.c_void_p, C.c_int, C.c_int]),
  "xotb200_load_shard": (C.c_int, [C.c_void_p, C.c_char_p, C.c_int, C.c_int]),
  "xotb200_load_tensor": (C.c_int, [C.c_void_p, C.c_char_p, C.c_void_p, C.POINTER(C.c_int64), C.c_int]),
  "xotb200_init_synthetic": (C.c_int, [C.c_void_p, C.c_uint64]),
  "xotb200_check_loaded": (C.c_int, [C.c_void_p]),
  "xotb200_begin_request": (C.c_int, [C.c_void_p, C.c_int]),
  "xotb200_begin_batch": (C.c_int, [C.c_void_p, C.c_int, C.c_int]),
  "xotb200_select_request": (C.c_int, [C.c_void_p, C.c_int]),
  "xotb200_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
  "xotb200_forward_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
  "xotb200_forward_hop": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.POINTER(C.c_int64), C.c_void_p]),
  "xotb200_last_token": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32)]),
  "xotb200_inbox_export": (C.c_int, [C.c_void_p, C.c_void_p]),
  "xotb200_link_next_ipc": (C.c_int, [C.c_void_p, C.c_void_p]),
  "xotb200_link_next_local": (C.c_int, [C.c_void_p, C.c_void_p]),
  "xotb200_post_to_next": (C.c_int, [C.c_void_p, C.c_int]),
  "xotb200_ring_launch": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int]),
  "xotb200_ring_launch_slots": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int]),
  "xotb200_post_token": (C.c_int, [C.c_void_p, C.c_int, C.c_int32, C.c_int]),
  "xotb200_ring_poll": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_int)]),
  "xotb200_clear_request": (C.c_int, [C.c_void_p, C.c_int]),
  "xotb200_ring_wait": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_float)]),
  "xotb200_ring_next_step": (C.c_int, [C.c_void_p, C.POINTER(C.c_int)]),
  "xotb200_ring_timestamps": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]),
  "xotb200_set_cta_limit": (C.c_int, [C.c_void_p, C.c_int]),
  "xotb200_set_prefill_mode": (C.c_int, [C.c_void_p, C.c_int]),
  "xotb200_debug_gemm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
  "xotb200_debug_routing": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.c_int]),
  "xotb200_debug_timeline": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int]),
  "xotb200_kernel_launches": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64)]),
  "xotb200_load_stats": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_double), C.POINTER(C.c_double)]),
  "xotb200_weight_bytes": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64)]),
  "xotb200_step_bytes": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_int64)]),
}

EXPORTED_SYMBOLS = tuple(_SIGS.keys())


def load(path: os.PathLike | None = None) -> C.CDLL:
  """dlopen the library (once) and declare every prototype of include/xotb200.h.  Raises if it is missing."""
  global _lib
  if _lib is not None and path is None:
    return _lib
  p = Path(path) if path else Path(os.environ.get("XOTB200_LIB", LIB_PATH))   # XOTB200_LIB: A/B-test another build
  if not p.exists():
    raise ImportError(f"{p} not found: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                      f"or `make -C xotorch_b200/csrc` — xotorch_b200 has no CPU fallback")
  lib = C.CDLL(str(p))
  for name, (res, args) in _SIGS.items():
    fn = getattr(lib, name)          # AttributeError if the library does not export a declared symbol
    fn.restype, fn.argtypes = res, args
  if path is None:
    _lib = lib
  return lib


# ---- libxotb200_lm.so: the layered-model engine (include/xotb200_lm.h) --------------------------------------------------
LM_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libxotb200_lm.so"
LM_DTYPE_BF16, LM_DTYPE_F32 = 0, 2
LM_MIX_LATENT_ATTN, LM_MIX_DELTA_RULE, LM_MIX_ATTENTION, LM_MIX_GATED_DELTA, LM_MIX_MATRIX_LSTM, LM_MIX_MAMBA2 = 0, 1, 2, 3, 4, 5
LM_FF_RELU2, LM_FF_XIELU, LM_FF_MOE, LM_FF_GELU = 0, 1, 2, 3
LM_EXPERT_SILU_GATED, LM_EXPERT_RELU2 = 0, 1
LM_ROUTER_SOFTMAX_ALL, LM_ROUTER_TOPK_SOFTMAX = 0, 1
LM_BLOCK_GROUP_RMS, LM_BLOCK_POST_LN, LM_BLOCK_POST_RMS, LM_BLOCK_PRE_SCALAR = 0, 1, 2, 3
LM_QKNORM_NONE, LM_QKNORM_HEAD, LM_QKNORM_ROW, LM_QKNORM_HEAD_PLAIN = 0, 1, 2, 3
LM_ROT_INTERLEAVED, LM_ROT_HALF = 0, 1


class LmLayer(C.Structure):
  """xotb200_lm_layer: one layer of a layered model (mixer kind, its sizes and constants, feed-forward size)"""
  _fields_ = [
    ("mixer", C.c_int32), ("heads", C.c_int32), ("dim", C.c_int32), ("vdim", C.c_int32), ("rot_dim", C.c_int32),
    ("kv_rank", C.c_int32), ("q_rank", C.c_int32), ("rot_dims", C.c_int32), ("rot_layout", C.c_int32), ("window", C.c_int32),
    ("out_gate", C.c_int32), ("low_rank", C.c_int32), ("ff", C.c_int32), ("rot_base", C.c_float), ("scale", C.c_float),
    ("kv_heads", C.c_int32), ("kv_from", C.c_int32), ("chunk", C.c_int32), ("qk_norm", C.c_int32), ("proj_bias", C.c_int32),
    ("dist_bias", C.c_int32), ("conv_taps", C.c_int32), ("ff_kind", C.c_int32), ("experts", C.c_int32), ("expert_ff", C.c_int32),
    ("top", C.c_int32), ("groups", C.c_int32), ("groups_keep", C.c_int32), ("softcap", C.c_float),
    ("out_bias", C.c_int32), ("sink", C.c_int32), ("rel_buckets", C.c_int32), ("rel_max", C.c_float), ("q_temp_coef", C.c_float),
    ("q_temp_every", C.c_int32), ("expert_act", C.c_int32), ("router_kind", C.c_int32), ("router_bias", C.c_int32),
    ("shared_ff", C.c_int32),
    ("rot_scale_factor", C.c_float), ("rot_scale_low", C.c_float), ("rot_scale_high", C.c_float), ("rot_scale_original", C.c_float),
    ("keep_first", C.c_int32), ("pool", C.c_int32), ("gate_cap", C.c_float), ("out_norm_groups", C.c_int32),
    ("par_on", C.c_int32), ("par_mixer", C.c_int32), ("par_heads", C.c_int32), ("par_kv_heads", C.c_int32), ("par_dim", C.c_int32),
    ("par_vdim", C.c_int32), ("par_conv_taps", C.c_int32), ("par_out_norm_groups", C.c_int32), ("par_gate_cap", C.c_float),
    ("mix_scale", C.c_float), ("par_scale", C.c_float),
  ]


class LmCfg(C.Structure):
  _fields_ = [
    ("n_layers", C.c_int32), ("start_layer", C.c_int32), ("end_layer", C.c_int32), ("width", C.c_int32), ("vocab", C.c_int32),
    ("norm_groups", C.c_int32), ("dtype", C.c_int32), ("norm_eps", C.c_float), ("block", C.c_int32), ("max_positions", C.c_int32),
    ("pos_sinusoid", C.c_int32), ("sinusoid_base", C.c_float), ("embed_norm", C.c_int32), ("logit_scale", C.c_float),
    ("logit_softcap", C.c_float), ("streams", C.c_int32), ("canon_taps", C.c_int32), ("residual_mult", C.c_float),
  ]


_I32P = C.POINTER(C.c_int32)
_LM_SIGS = {
  "xotb200_lm_last_error": (C.c_char_p, []),
  "xotb200_lm_version": (C.c_char_p, []),
  "xotb200_lm_create": (C.c_int, [C.POINTER(LmCfg), C.POINTER(LmLayer), C.c_int, C.POINTER(C.c_void_p)]),
  "xotb200_lm_destroy": (C.c_int, [C.c_void_p]),
  "xotb200_lm_load_dir": (C.c_int, [C.c_void_p, C.c_char_p]),
  "xotb200_lm_load_tensor": (C.c_int, [C.c_void_p, C.c_char_p, C.c_void_p, C.POINTER(C.c_int64), C.c_int]),
  "xotb200_lm_check_loaded": (C.c_int, [C.c_void_p]),
  "xotb200_lm_init_synthetic": (C.c_int, [C.c_void_p, C.c_uint64]),
  "xotb200_lm_begin": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int]),
  "xotb200_lm_clear_request": (C.c_int, [C.c_void_p, C.c_int]),
  "xotb200_lm_request_len": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_int)]),
  "xotb200_lm_step": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p,
                                C.c_void_p, C.c_void_p]),
  "xotb200_lm_set_trace": (C.c_int, [C.c_void_p, C.c_int]),
  "xotb200_lm_read_trace": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64]),
  "xotb200_lm_set_gemm_mode": (C.c_int, [C.c_void_p, C.c_int]),
  "xotb200_lm_kernel_launches": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64)]),
  "xotb200_lm_set_graphs": (C.c_int, [C.c_void_p, C.c_int]),
  "xotb200_lm_graph_replays": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64)]),
  "xotb200_lm_set_attention_mode": (C.c_int, [C.c_void_p, C.c_int]),
  "xotb200_lm_prompt_attention_launches": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64)]),
  "xotb200_lm_tensor_core_launches": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64)]),
  "xotb200_lm_weight_bytes": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64)]),
  "xotb200_lm_cache_stats": (C.c_int, [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]),
  "xotb200_lm_last_step_ms": (C.c_int, [C.c_void_p, C.POINTER(C.c_float)]),
}
LM_EXPORTED_SYMBOLS = tuple(_LM_SIGS.keys())
_lm_lib = None


def load_lm(path: os.PathLike | None = None, build: bool = True) -> C.CDLL:
  """dlopen libxotb200_lm.so (once).  In a checkout that has not been built yet the library is compiled first — only this one
  (`make lm`, a few seconds of nvcc), not the shard engine's persistent kernels; a library older than its sources is rebuilt
  when the tree is writable.  Raises if it cannot be had: no CPU fallback."""
  global _lm_lib
  if _lm_lib is not None and path is None:
    return _lm_lib
  p = Path(path) if path else Path(os.environ.get("XOTB200_LM_LIB", LM_LIB_PATH))
  if build and path is None and "XOTB200_LM_LIB" not in os.environ:
    src = Path(__file__).resolve().parent / "csrc"
    deps = [src / n for n in ("layered.cu", "layered_kernels.cuh", "layered_blocks.cuh", "layered_gqa.cuh", "layered_tc.cuh", "prefill_tc.cuh", "kernels.cuh", "st_header.h")]
    deps.append(src.parent.parent / "include" / "xotb200_lm.h")
    stale = p.exists() and any(d.exists() and d.stat().st_mtime > p.stat().st_mtime for d in deps)
    if not p.exists() or stale:
      import subprocess
      r = subprocess.run(["make", "-C", str(src), "lm"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
      if r.returncode != 0 and not p.exists():
        raise ImportError(f"building {p} failed:\n{r.stdout[-4000:]}")
  if not p.exists():
    raise ImportError(f"{p} not found: build it with `make -C xotorch_b200/csrc lm` — xotorch_b200 has no CPU fallback")
  lib = C.CDLL(str(p))
  for name, (res, args) in _LM_SIGS.items():
    fn = getattr(lib, name)
    fn.restype, fn.argtypes = res, args
  if path is None:
    _lm_lib = lib
  return lib


def check_lm(rc: int) -> int:
  if rc < 0:
    raise XotB200Error(rc, load_lm().xotb200_lm_last_error().decode("utf-8", "replace"))
  return rc


def check(rc: int) -> int:
  if rc < 0:
    raise XotB200Error(rc, load().xotb200_last_error().decode("utf-8", "replace"))
  return rc
