"""The engine's device operations: thin checked wrappers over the sm_100a kernel libraries.

Every function writes into tensors the caller passes, runs on the current CUDA stream and
allocates nothing, so that a step can be captured in a CUDA graph.  There is no other
implementation behind these names: if the libraries cannot be built or loaded, or a tensor is not
on a CUDA device, the call raises.

Large-M bf16 matrix products go to cuBLAS through ``torch.matmul`` - the reference uses the same
library for all of its products (miniinfer/layers/linear.py:30-32); everything else is this
package's own CUDA.
"""

from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional

import torch

from . import build

F32, BF16 = 0, 1
PREFILL_TILE = 64     # query rows of one tile of the prefill attention kernels
PREFILL_WIDE_TILE = 128   # tokens of a work of the tcgen05 prefill kernel when a block (or each block of a pair) takes one head
PREFILL_PAIRS_MIN_WIDE_TILES = 48   # steps with at least this many such tiles (6144 new tokens) let two blocks share a work
SKINNY_MAX_M = 64     # the most rows the skinny kernel takes
SKINNY_BEST_M = 16    # up to here it is the faster one; above, cuBLAS is (measured on B200, M = 32 and 64)
# Rows from which the tcgen05 gate-up product with SwiGLU in its epilogue beats the library product followed by the
# activation kernel.  Device times on B200 with a cold L2 (each call recorded into a CUDA graph behind a 256 MB flush),
# library + activation against the fused kernel, at 64 / 512 / 1024 / 1280 / 2048 rows:
#   K = 1024, I = 3072:    7.1 / 11.9 / 17.1 / 19.9 / 28.9 us   against   13.7 / 14.9 / 20.5 / 21.0 / 27.0 us
#   K = 2048, I = 6144:   15.4 / 25.6 / 44.2 / 54.0 / 81.7 us   against   21.4 / 34.0 / 45.4 / 56.3 / 77.4 us
#   K = 4096, I = 12288:  49.6 / 76.1 / 142 / 190 / 284 us      against   63.6 / 84.4 / 149 / 173 / 270 us
# The fused kernel saves the pass over [M, 2I] but needs about 13 us to fill and drain its pipeline of 256-row tiles,
# so for prompt portions and mixed steps of fewer rows the library stays (blocks that work alone on 128-row tiles,
# MINIINFER_B200_GEMM_TC=1, are slower still).
GEMM_TC_MIN_M = 1280        # for K >= 4096
GEMM_TC_MIN_M_NARROW = 1792  # for narrower models
_MM_F32_OUT: Optional[bool] = None   # whether torch.mm writes float32 from bf16 operands into a given tensor


class KernelError(RuntimeError):
  """A kernel refused its arguments or failed to launch."""


_libs: Dict[str, ctypes.CDLL] = {}


def _load(name: str, path: str) -> ctypes.CDLL:
  lib = ctypes.CDLL(path)
  lib.mi_last_error.restype = ctypes.c_char_p
  _libs[name] = lib
  return lib


def common_lib() -> ctypes.CDLL:
  lib = _libs.get("common")
  if lib is None:
    lib = _load("common", build.build_common())
  return lib


def attention_lib(head_dim: int) -> ctypes.CDLL:
  name = f"attn_hd{head_dim}"
  lib = _libs.get(name)
  if lib is None:
    lib = _load(name, build.build_attention(head_dim))
  return lib


def loaded_libraries() -> Dict[str, str]:
  return {k: v._name for k, v in _libs.items()}


_launches = 0


def launch_count() -> int:
  """Kernels of this package launched so far by this process (launches recorded into a CUDA graph
  are counted once, when they are recorded)."""
  return _launches


def _check(lib: ctypes.CDLL, code: int, kernels: int = 1) -> None:
  global _launches
  if code != 0:
    raise KernelError(lib.mi_last_error().decode())
  _launches += kernels


def _dt(t: torch.Tensor) -> int:
  if t.dtype == torch.float32:
    return F32
  if t.dtype == torch.bfloat16:
    return BF16
  raise KernelError(f"dtype {t.dtype} is not supported (float32 or bfloat16)")


def _ptr(t: Optional[torch.Tensor], dtype: Optional[torch.dtype] = None) -> ctypes.c_void_p:
  if t is None:
    return ctypes.c_void_p(0)
  if not t.is_cuda:
    raise KernelError("the engine's kernels run on CUDA tensors only (got a CPU tensor)")
  if not t.is_contiguous():
    raise KernelError("kernel arguments must be contiguous")
  if dtype is not None and t.dtype != dtype:
    raise KernelError(f"expected {dtype}, got {t.dtype}")
  return ctypes.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> ctypes.c_void_p:
  """The current CUDA stream of the current device (also the capture stream while a graph is recorded)."""
  if _raw_stream is not None:
    return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
  return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


# --------------------------------------------------------------------------------------------


def embedding(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, scale: float = 1.0, copies: int = 1) -> None:
  """out[t] = scale * table[ids[t]] as float32, ``copies`` times side by side in a row of out.  ids: int32, already
  checked to lie in the vocabulary."""
  lib = common_lib()
  T, H = out.shape[0], table.shape[1]
  if out.shape[1] != H * copies or ids.shape[0] != T or copies < 1:
    raise KernelError("embedding: shapes do not match")
  _check(lib, lib.mi_embedding(_ptr(out, torch.float32), _ptr(table), _dt(table), _ptr(ids, torch.int32),
                               T, H, ctypes.c_float(scale), int(copies), _stream()))


def add_layernorm(out: torch.Tensor, resid: torch.Tensor, delta: Optional[torch.Tensor], delta2: Optional[torch.Tensor],
                  weight: torch.Tensor, bias: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None,
                  write_back: bool = True) -> None:
  """out[r] = (s - mean(s)) / sqrt(var(s) + eps) * weight + bias with s = resid[row] + (delta[row] + delta2[row]), both
  deltas optional and of one dtype; the sum goes back to resid if write_back.  All in float32."""
  lib = common_lib()
  R, H = out.shape
  if resid.shape[1] != H or weight.shape != (H,) or bias.shape != (H,):
    raise KernelError("add_layernorm: shapes do not match")
  for d in (delta, delta2):
    if d is not None and d.shape != resid.shape:
      raise KernelError("add_layernorm: a delta differs from the residual in shape")
  if delta is not None and delta2 is not None and delta.dtype != delta2.dtype:
    raise KernelError("add_layernorm: the two deltas differ in dtype")
  if (rows is None and resid.shape[0] != R) or (rows is not None and rows.shape[0] != R):
    raise KernelError("add_layernorm: out, rows and resid differ in rows")
  first = delta if delta is not None else delta2
  _check(lib, lib.mi_add_layernorm(_ptr(out), _dt(out), _ptr(resid, torch.float32), _ptr(delta), _ptr(delta2),
                                   _dt(first) if first is not None else F32, _ptr(weight, torch.float32), _ptr(bias, torch.float32),
                                   _ptr(rows, torch.int32) if rows is not None else _ptr(None), R, H,
                                   ctypes.c_float(eps), int(bool(write_back)), _stream()))


def add_rmsnorm(out: torch.Tensor, resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                eps: float, rows: Optional[torch.Tensor] = None, write_back: bool = True) -> None:
  """out[r] = weight * norm(resid[row] + delta[row]); the sum goes back to resid if write_back."""
  lib = common_lib()
  R, H = out.shape
  if resid.shape[1] != H or weight.shape[0] != H or (delta is not None and delta.shape != resid.shape):
    raise KernelError("add_rmsnorm: shapes do not match")
  if rows is None and resid.shape[0] != R:
    raise KernelError("add_rmsnorm: out and resid differ in rows")
  if rows is not None and rows.shape[0] != R:
    raise KernelError("add_rmsnorm: rows and out differ in length")
  _check(lib, lib.mi_add_rmsnorm(_ptr(out), _dt(out), _ptr(resid, torch.float32), _ptr(delta),
                                 _dt(delta) if delta is not None else F32, _ptr(weight, torch.float32),
                                 _ptr(rows, torch.int32) if rows is not None else _ptr(None), R, H,
                                 ctypes.c_float(eps), int(bool(write_back)), _stream()))


_transposed_views: Dict[int, tuple] = {}
_capturing = False


class recording_graph:
  """``with ops.recording_graph():`` around a stream capture: library products then go through
  PyTorch, whose cuBLAS handle has a workspace that is safe to use while a graph is recorded."""

  def __enter__(self):
    global _capturing
    self._before = _capturing
    _capturing = True
    return self

  def __exit__(self, *exc):
    global _capturing
    _capturing = self._before
    return False



def _transposed(w: torch.Tensor) -> torch.Tensor:
  """``w.t()``, kept per weight tensor: making the view costs more host time than a small product."""
  hit = _transposed_views.get(id(w))
  if hit is not None and hit[0] is w:
    return hit[1]
  if len(_transposed_views) > 4096:
    _transposed_views.clear()
  v = w.t()
  _transposed_views[id(w)] = (w, v)
  return v


def _mm_f32_out_works(device) -> bool:
  """Tried once: bf16 x bf16 -> float32 through cuBLAS, written into a tensor the caller owns."""
  global _MM_F32_OUT
  if _MM_F32_OUT is None:
    try:
      a = torch.ones(32, 16, dtype=torch.bfloat16, device=device)
      o = torch.empty(32, 32, dtype=torch.float32, device=device)
      torch.mm(a, a.t(), out_dtype=torch.float32, out=o)
      _MM_F32_OUT = bool((o == 16).all().item())
    except (TypeError, RuntimeError, NotImplementedError):
      _MM_F32_OUT = False
  return _MM_F32_OUT


def linear(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, force_skinny: bool = False, force_stream: bool = False) -> None:
  """out[M, N] = x[M, K] @ w[N, K]^T.  float32 operands: this package's fp32 FMA kernel (out float32).
  bfloat16 operands: for M <= 16 the weight-streaming kernels (out bf16 or fp32; a row's value does not depend
  on the other rows) - the tcgen05 one from ``STREAM_TC_MIN_BYTES`` of weights on, the mma.sync one below -,
  cuBLAS above 16 rows (where the reference uses it for every product).
  ``force_skinny``: the mma.sync kernel for any M (in slices of 64 rows); ``force_stream``: the tcgen05 one at any size."""
  M, K = x.shape
  N = w.shape[0]
  if w.shape[1] != K or out.shape != (M, N):
    raise KernelError(f"linear: shapes do not match: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
  if M == 0:
    return
  lib = common_lib()
  if not x.is_contiguous() or (x.dtype == torch.bfloat16 and (K % 8 != 0 or x.data_ptr() % 16 != 0 or w.data_ptr() % 16 != 0)):
    # x is a column range of wider rows, or its rows cannot be read 16 bytes at a time: the library product for many
    # bfloat16 rows, else the product that takes any strides and sizes
    if x.dim() != 2 or x.stride(1) != 1 or x.dtype != w.dtype:
      raise KernelError("linear: x must have contiguous rows of the weights' dtype")
    lda = int(x.stride(0))
    if (x.dtype == torch.bfloat16 and M > SKINNY_BEST_M and K % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
        and out.dtype in (torch.bfloat16, torch.float32) and out.is_contiguous()):
      if not _capturing:
        _check(lib, lib.mi_gemm_cublas_bf16(_ptr(out), _dt(out), ctypes.c_void_p(x.data_ptr()), _ptr(w), M, N, K, lda, _stream()), kernels=0)
        return
      if out.dtype == torch.bfloat16:
        torch.mm(x, _transposed(w), out=out)
        return
      if _mm_f32_out_works(out.device):
        torch.mm(x, _transposed(w), out_dtype=torch.float32, out=out)
        return
    linear_batched(out.unsqueeze(1), x.unsqueeze(1), w.unsqueeze(0))
    return
  if x.dtype == torch.float32:
    _check(lib, lib.mi_gemm_f32(_ptr(out, torch.float32), _ptr(x), _ptr(w, torch.float32), M, N, K, N, _stream()))
    return
  if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
    raise KernelError(f"linear: operands must both be float32 or both bfloat16, got {x.dtype} and {w.dtype}")
  if _streams(M, N, K, force_skinny, force_stream) and out.dtype in (torch.bfloat16, torch.float32):
    parts, counters, status = _stream_workspace(lib, x.device)
    _check(lib, lib.mi_gemm_stream_tc_bf16(_ptr(out), _dt(out), _ptr(x), _ptr(w), M, N, K, N, _ptr(parts, torch.float32),
                                           _ptr(counters, torch.int32), counters.numel(), parts.shape[0],
                                           _ptr(status, torch.int32), _stream()))
    return
  if M <= SKINNY_BEST_M or (force_skinny and M <= SKINNY_MAX_M):
    _check(lib, lib.mi_gemm_skinny_bf16(_ptr(out), _dt(out), _ptr(x), _ptr(w), M, N, K, N, _stream()))
    return
  if not force_skinny:
    if not (out.is_cuda and out.is_contiguous() and x.is_contiguous() and w.is_contiguous()):
      raise KernelError("linear: operands and out must be contiguous CUDA tensors")
    if K % 8 != 0:
      raise KernelError(f"linear: K={K} must be a multiple of 8 (16-byte loads of bf16 rows)")
    if not _capturing and out.dtype in (torch.bfloat16, torch.float32):
      # more than 16 rows: straight to cuBLAS (a third of the host time of torch.mm); not while a graph is recorded
      _check(lib, lib.mi_gemm_cublas_bf16(_ptr(out), _dt(out), _ptr(x), _ptr(w), M, N, K, K, _stream()), kernels=0)
      return
    if out.dtype == torch.bfloat16:
      torch.mm(x, _transposed(w), out=out)
      return
    if out.dtype == torch.float32 and _mm_f32_out_works(out.device):
      torch.mm(x, _transposed(w), out_dtype=torch.float32, out=out)
      return
  for m0 in range(0, M, SKINNY_MAX_M):
    m1 = min(M, m0 + SKINNY_MAX_M)
    _check(lib, lib.mi_gemm_skinny_bf16(_ptr(out[m0:m1]), _dt(out), _ptr(x[m0:m1]), _ptr(w), m1 - m0, N, K, N,
                                        _stream()))


# Few rows times a large weight matrix: the tcgen05 kernel that deals the matrix out to the SMs in equal stretches
# (gemm_stream_tc.cu) from 160 MiB of weights on, and from 80 MiB where the matrix has more than 4096 rows; else the
# mma.sync kernel (gemm_skinny.cu), whose launches start and end faster and whose 16-warp blocks fill the SMs in one
# round for up to 4096 rows.  Measured on B200, 8 rows, cold weights, microseconds (tcgen05 / mma.sync):
#   10240 x 5120 (105 MB) 23.6 / 26.1    5120 x 8192 (84 MB) 19.9 / 21.1    5120 x 25600 (262 MB) 49.2 / 64.1
#   SwiGLU 2 x 25600 x 5120 (524 MB) 84.3 / 93.4    SwiGLU 2 x 12288 x 4096 (201 MB) 38.8 / 41.7
#   151936 x 1024 (311 MB) 55.1 / 56.2    4096 x 12288 (101 MB) 23.1 / 19.7    6144 x 4096 (50 MB) 14.2 / 11.7
STREAM_TC_MIN_BYTES = 160 << 20
STREAM_TC_MIN_BYTES_MANY_ROWS = 80 << 20
STREAM_TC_MAX_TILES = 1 << 14
_stream_ws: Dict[int, tuple] = {}


def _streams(M: int, weight_rows: int, K: int, force_skinny: bool, force_stream: bool) -> bool:
  if M > SKINNY_BEST_M or force_skinny or K < 64 or K % 8 != 0:
    return False
  mode = os.environ.get("MINIINFER_B200_GEMM_STREAM", "")
  if mode == "0":
    return False
  size = 2 * weight_rows * K
  return (force_stream or mode == "1" or size >= STREAM_TC_MIN_BYTES
          or (size >= STREAM_TC_MIN_BYTES_MANY_ROWS and weight_rows > 4096))


def _stream_workspace(lib, device):
  """Partial sums, tile counters and the status word of the tcgen05 streaming product, made once per device."""
  idx = device.index if device.index is not None else torch.cuda.current_device()
  ws = _stream_ws.get(idx)
  if ws is None:
    if torch.cuda.is_current_stream_capturing():
      raise KernelError("gemm_stream_tc: its workspace must exist before a graph is recorded (run the step once before)")
    floats, blocks = ctypes.c_longlong(0), ctypes.c_int(0)
    _check(lib, lib.mi_gemm_stream_tc_workspace(ctypes.byref(floats), ctypes.byref(blocks)), kernels=0)
    parts = torch.zeros((blocks.value, floats.value // blocks.value), dtype=torch.float32, device=device)
    counters = torch.zeros(STREAM_TC_MAX_TILES, dtype=torch.int32, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    ws = _stream_ws[idx] = (parts, counters, status)
  return ws


def fuses_few_rows(x_rows: int, dtype: torch.dtype) -> bool:
  """Whether a step of ``x_rows`` rows takes the few-row products with the norm and the residual add fused to them
  (six launches per layer instead of eight).  Off unless MINIINFER_B200_FUSE_FEW_ROWS=1: measured on B200 (Qwen3-0.6B
  shape) the fused decode step takes 1.05 ms against 0.99 ms at batch 8 and 0.78 against 0.74 ms at batch 1.  The
  norm kernels between the products are where, under dependent launch, the next product's blocks get onto the SMs
  and fetch their weights - a step from which the norm launches are simply left out is slower, not faster - while a
  product that follows a product directly finds the SMs' registers taken until its predecessor has ended."""
  return dtype == torch.bfloat16 and 0 < x_rows <= SKINNY_BEST_M and os.environ.get("MINIINFER_B200_FUSE_FEW_ROWS", "0") == "1"


def linear_normed(out: torch.Tensor, resid: torch.Tensor, norm_weight: torch.Tensor, eps: float, w: torch.Tensor) -> None:
  """out[M, N] = rmsnorm(resid)[M, K] @ w[N, K]^T for up to 16 rows: the norm in the product's prologue.
  resid float32, w and out bfloat16; the normalised rows are rounded to bfloat16 once, as ``add_rmsnorm`` rounds them."""
  M, K = resid.shape
  N = w.shape[0]
  if w.shape[1] != K or out.shape != (M, N) or norm_weight.shape != (K,):
    raise KernelError(f"linear_normed: shapes do not match: resid {tuple(resid.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
  lib = common_lib()
  _check(lib, lib.mi_gemm_skinny_norm_bf16(_ptr(out, torch.bfloat16), _ptr(resid, torch.float32), _ptr(norm_weight, torch.float32),
                                           ctypes.c_float(eps), _ptr(w, torch.bfloat16), M, N, K, N, _stream()))


def linear_swiglu_normed(out: torch.Tensor, resid: torch.Tensor, norm_weight: torch.Tensor, eps: float, w: torch.Tensor) -> None:
  """out[M, I] = silu(n @ w[:I]^T) * (n @ w[I:]^T) with n = rmsnorm(resid), for up to 16 rows, in one kernel."""
  M, K = resid.shape
  I = out.shape[1]
  if w.shape != (2 * I, K) or out.shape[0] != M or norm_weight.shape != (K,):
    raise KernelError(f"linear_swiglu_normed: shapes do not match: resid {tuple(resid.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
  lib = common_lib()
  _check(lib, lib.mi_gemm_skinny_norm_swiglu_bf16(_ptr(out, torch.bfloat16), _ptr(resid, torch.float32), _ptr(norm_weight, torch.float32),
                                                  ctypes.c_float(eps), _ptr(w, torch.bfloat16), M, I, K, I, _stream()))


def linear_add(resid: torch.Tensor, x: torch.Tensor, w: torch.Tensor) -> None:
  """resid[M, N] += bfloat16(x[M, K] @ w[N, K]^T) for up to 16 rows: the residual add in the product's epilogue.
  The product is rounded to bfloat16 before it is added, as it is when a bfloat16 product is handed to ``add_rmsnorm``."""
  M, K = x.shape
  N = w.shape[0]
  if w.shape[1] != K or resid.shape != (M, N):
    raise KernelError(f"linear_add: shapes do not match: x {tuple(x.shape)}, w {tuple(w.shape)}, resid {tuple(resid.shape)}")
  lib = common_lib()
  _check(lib, lib.mi_gemm_skinny_add_f32(_ptr(resid, torch.float32), _ptr(x, torch.bfloat16), _ptr(w, torch.bfloat16), M, N, K, N, _stream()))


def qk_norm_rope_store(qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                       cos_sin: Optional[torch.Tensor], positions: torch.Tensor,
                       slot_mapping: Optional[torch.Tensor], kv_layer: Optional[torch.Tensor],
                       num_heads: int, num_kv_heads: int, head_dim: int, eps: float) -> None:
  """In place on the fused QKV rows: per-head RMSNorm of q and k, rotary encoding from the table,
  and the store of k and v into the layer's pages at ``slot_mapping`` (page * page_size + offset)."""
  lib = common_lib()
  T = qkv.shape[0]
  if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
    raise KernelError("qk_norm_rope_store: qkv width does not match the head counts")
  rotary_dim = 0
  if cos_sin is not None:
    rotary_dim = cos_sin.shape[1]
  page_size = 0
  if kv_layer is not None:
    if kv_layer.dtype != qkv.dtype:
      raise KernelError("qk_norm_rope_store: cache and activations differ in dtype")
    if kv_layer.shape[1:] != (2, num_kv_heads, kv_layer.shape[3], head_dim):
      raise KernelError(f"qk_norm_rope_store: cache layer has shape {tuple(kv_layer.shape)}")
    page_size = kv_layer.shape[3]
  _check(lib, lib.mi_qk_norm_rope_store(
    _ptr(qkv), _dt(qkv), _ptr(q_weight, torch.float32) if q_weight is not None else _ptr(None),
    _ptr(k_weight, torch.float32) if k_weight is not None else _ptr(None),
    _ptr(cos_sin, torch.float32) if cos_sin is not None else _ptr(None), rotary_dim,
    _ptr(positions, torch.int32), _ptr(slot_mapping, torch.int32) if slot_mapping is not None else _ptr(None),
    _ptr(kv_layer), T, num_heads, num_kv_heads, head_dim, page_size, ctypes.c_float(eps), _stream()))


def qkv_norm_mix_store(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, q_out: torch.Tensor, num_heads: int,
                       num_kv_heads: int, dim: int, vdim: int, eps: float, normalise: bool = True,
                       q_weight: Optional[torch.Tensor] = None, k_weight: Optional[torch.Tensor] = None,
                       mix: Optional[torch.Tensor] = None, v_other: Optional[torch.Tensor] = None, v_mode: int = 0,
                       slot_mapping: Optional[torch.Tensor] = None, kv_layer: Optional[torch.Tensor] = None,
                       rope: Optional[torch.Tensor] = None, positions: Optional[torch.Tensor] = None,
                       interleaved: bool = False, bias: Optional[torch.Tensor] = None, norm_whole: bool = False) -> None:
  """From the rows of a fused projection (queries at column ``q_off``, keys at ``k_off``, values at ``v_off``) to what
  attention reads, for heads that are not rotated: query and key heads divided by their root mean square over
  ``dim`` (x / sqrt(mean(x^2) + eps), float32; times ``q_weight`` / ``k_weight`` if given); queries into
  ``q_out [tokens, heads, cache head size]`` padded with zeros; values mixed with another layer's values of the same
  token (``v_mode`` 2: v <- (1 - mix) v + mix v_other, ``mix`` a scalar on the device), recorded as those values
  (``v_mode`` 1) or left alone (0); keys and values stored into the layer's pages at ``slot_mapping``.
  ``rope [positions, rot_dims]`` float32 (cos of rot_dims / 2 angles, then their sines): the first ``rot_dims`` values of
  every query and key head are rotated, after the norm, by the angles of the token's position - value i with value
  i + rot_dims / 2, or 2i with 2i + 1 if ``interleaved``.  ``v_off == k_off`` makes the values the keys as projected.
  ``bias`` float32, indexed like the projection's columns and covering the queries, keys and values, is added first.  ``norm_whole``: the root
  mean square runs over all query heads of a token at once (and over all its key heads), and ``q_weight`` / ``k_weight``
  hold a value per head and dimension (``[heads * dim]``, ``[kv heads * dim]``)."""
  lib = common_lib()
  T = proj.shape[0]
  hdp = q_out.shape[1] // num_heads
  if bias is not None and (bias.dim() != 1 or bias.shape[0] < max(q_off + num_heads * dim, k_off + num_kv_heads * dim, v_off + num_kv_heads * vdim)):
    raise KernelError("qkv_norm_mix_store: the bias must have a value for every query, key and value column of the projection")
  for wt, n in ((q_weight, num_heads), (k_weight, num_kv_heads)):
    if wt is not None and wt.shape != ((n * dim,) if norm_whole else (dim,)):
      raise KernelError("qkv_norm_mix_store: a norm weight does not match the span of its norm")
  if q_out.shape != (T, num_heads * hdp) or q_out.dtype != proj.dtype:
    raise KernelError("qkv_norm_mix_store: q_out does not match the projection rows")
  width = proj.shape[1]
  if max(q_off + num_heads * dim, k_off + num_kv_heads * dim, v_off + num_kv_heads * vdim) > width:
    raise KernelError("qkv_norm_mix_store: the heads do not fit the projection rows")
  page_size = 0
  if kv_layer is not None:
    if kv_layer.dtype != proj.dtype or kv_layer.dim() != 5 or kv_layer.shape[1:3] != (2, num_kv_heads) or kv_layer.shape[4] != hdp:
      raise KernelError(f"qkv_norm_mix_store: cache layer has shape {tuple(kv_layer.shape)}, head size {hdp} expected")
    page_size = kv_layer.shape[3]
  if v_mode and (v_other is None or v_other.shape != (T, num_kv_heads * vdim) or v_other.dtype != proj.dtype):
    raise KernelError("qkv_norm_mix_store: the other layer's values must be [tokens, kv heads * vdim] in the rows' dtype")
  none = _ptr(None)
  _check(lib, lib.mi_qkv_norm_mix_store(
    _ptr(proj), _dt(proj), width, q_off, k_off, v_off, T, num_heads, num_kv_heads, dim, vdim, hdp, _ptr(q_out),
    _ptr(q_weight, torch.float32) if q_weight is not None else none, _ptr(k_weight, torch.float32) if k_weight is not None else none,
    ctypes.c_float(eps), int(bool(normalise)), _ptr(mix, torch.float32) if mix is not None else none,
    _ptr(v_other) if v_other is not None else none, int(v_mode),
    _ptr(slot_mapping, torch.int32) if (slot_mapping is not None and kv_layer is not None) else none,
    _ptr(kv_layer) if kv_layer is not None else none, page_size,
    _ptr(rope, torch.float32) if rope is not None else none, _ptr(positions, torch.int32) if rope is not None else none,
    int(rope.shape[1]) if rope is not None else 0, int(bool(interleaved)),
    _ptr(bias, torch.float32) if bias is not None else none, int(bool(norm_whole)), _stream()))


def add_rmsnorm_pair(out1: torch.Tensor, out2: Optional[torch.Tensor], resid: torch.Tensor, delta: Optional[torch.Tensor],
                     delta2: Optional[torch.Tensor], w1: torch.Tensor, w2: Optional[torch.Tensor], eps: float,
                     rows: Optional[torch.Tensor] = None, write_back: bool = True) -> None:
  """s = resid[row] + (delta[row] + delta2[row]) (both optional, of one dtype); out1[r] = w1 * s / rms(s) and, if asked
  for, out2[r] = w2 * s / rms(s), rms(s) = sqrt(mean(s^2) + eps); the sum goes back to resid if write_back.  float32."""
  lib = common_lib()
  R, H = out1.shape
  if resid.shape[1] != H or w1.shape != (H,) or (out2 is not None and (w2 is None or w2.shape != (H,) or out2.shape != out1.shape or out2.dtype != out1.dtype)):
    raise KernelError("add_rmsnorm_pair: shapes do not match")
  for d in (delta, delta2):
    if d is not None and d.shape != resid.shape:
      raise KernelError("add_rmsnorm_pair: a delta differs from the residual in shape")
  if delta is not None and delta2 is not None and delta.dtype != delta2.dtype:
    raise KernelError("add_rmsnorm_pair: the two deltas differ in dtype")
  if (rows is None and resid.shape[0] != R) or (rows is not None and rows.shape[0] != R):
    raise KernelError("add_rmsnorm_pair: out, rows and resid differ in rows")
  first = delta if delta is not None else delta2
  _check(lib, lib.mi_add_rmsnorm_pair(_ptr(out1), _ptr(out2), _dt(out1), _ptr(resid, torch.float32), _ptr(delta), _ptr(delta2),
                                      _dt(first) if first is not None else F32, _ptr(w1, torch.float32),
                                      _ptr(w2, torch.float32) if w2 is not None else _ptr(None),
                                      _ptr(rows, torch.int32) if rows is not None else _ptr(None), R, H, ctypes.c_float(eps),
                                      int(bool(write_back)), _stream()))


def rms_pair_sum(out: torch.Tensor, a: torch.Tensor, b: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, eps: float, scale: float) -> None:
  """out = scale * (w1 * a / rms(a) + w2 * b / rms(b)) row by row, rms(x) = sqrt(mean(x^2) + eps), in float32."""
  lib = common_lib()
  R, H = out.shape
  if a.shape != (R, H) or b.shape != (R, H) or w1.shape != (H,) or w2.shape != (H,) or a.dtype != out.dtype or b.dtype != out.dtype:
    raise KernelError("rms_pair_sum: shapes or dtypes do not match")
  _check(lib, lib.mi_rms_pair_sum(_ptr(out), _ptr(a), _ptr(b), _dt(out), _ptr(w1, torch.float32), _ptr(w2, torch.float32), R, H,
                                  ctypes.c_float(eps), ctypes.c_float(scale), _stream()))


def _cols(t: torch.Tensor, what: str):
  """(pointer, row stride) of a 2-d operand that may be a column range of wider contiguous rows."""
  if t.dim() != 2 or t.stride(1) != 1 or not t.is_cuda:
    raise KernelError(f"{what}: operands must be CUDA matrices with contiguous rows")
  return ctypes.c_void_p(t.data_ptr()), int(t.stride(0))


def linear_batched(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, softplus: bool = False,
                   row_gate: Optional[torch.Tensor] = None) -> None:
  """out[:, b, :] = x[:, b, :] @ w[b]^T for ``x [M, batch, K]``, ``w [batch, N, K]``, ``out [M, batch, N]`` - views whose
  strides may be anything as long as the last axis is contiguous (the heads of a token's row, a column range of a
  row); float32 sums, k ascending.  ``bias [N]`` float32 is added, ``softplus`` applied, and with ``row_gate [M, >= batch]``
  (one logit per row and batch) the result is multiplied with its sigmoid."""
  lib = common_lib()
  M, B, K = x.shape
  N = w.shape[1]
  if w.shape != (B, N, K) or out.shape != (M, B, N) or x.dtype != w.dtype:
    raise KernelError(f"linear_batched: shapes do not match: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
  for t in (x, w, out):
    if t.stride(2) != 1 or not t.is_cuda:
      raise KernelError("linear_batched: the last axis of every operand must be contiguous, on a CUDA device")
  if M == 0:
    return
  gate_stride = 0
  if row_gate is not None:
    if row_gate.dim() != 2 or row_gate.shape[0] != M or row_gate.shape[1] < B or row_gate.stride(1) != 1 or row_gate.dtype != x.dtype:
      raise KernelError("linear_batched: the row gate must hold a logit per row and batch, in the operands' dtype")
    gate_stride = row_gate.stride(0)
  few = M <= 16 and x.dtype == torch.bfloat16
  _check(lib, (lib.mi_gemm_batched_few_rows if few else lib.mi_gemm_batched)(
    ctypes.c_void_p(out.data_ptr()), _dt(out), ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()), _dt(x), B, M, N, K,
    int(x.stride(0)), ctypes.c_longlong(x.stride(1)), int(w.stride(1)), ctypes.c_longlong(w.stride(0)),
    int(out.stride(0)), ctypes.c_longlong(out.stride(1)), _ptr(bias, torch.float32) if bias is not None else _ptr(None),
    int(bool(softplus)), ctypes.c_void_p(row_gate.data_ptr()) if row_gate is not None else _ptr(None), gate_stride, _stream()))


def linear_parts(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor) -> None:
  """A block-diagonal map: ``out[b] = x[:, b K:(b + 1) K] @ w[b]^T`` for ``x [M, parts * K]``, ``w [parts, N, K]`` and
  ``out [parts, M, N]`` (bfloat16 or float32), all contiguous.  bfloat16 with more than 16 rows: one strided batched library
  product on the tensor cores (a library product a part while a graph is recorded); else the batched FMA kernels."""
  B, N, K = w.shape
  M = x.shape[0]
  if x.shape != (M, B * K) or out.shape != (B, M, N) or x.dtype != w.dtype or not (x.is_contiguous() and w.is_contiguous() and out.is_contiguous()):
    raise KernelError(f"linear_parts: shapes do not match: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
  if M == 0:
    return
  if x.dtype == torch.bfloat16 and M > SKINNY_BEST_M and K % 8 == 0 and out.dtype in (torch.bfloat16, torch.float32):
    if not _capturing:
      lib = common_lib()
      _check(lib, lib.mi_gemm_cublas_bf16_batched(_ptr(out), _dt(out), _ptr(x), _ptr(w), M, N, K, B * K, ctypes.c_longlong(K),
                                                  ctypes.c_longlong(N * K), ctypes.c_longlong(M * N), B, _stream()), kernels=0)
      return
    # while a graph is recorded: torch's products, a part at a time (float32 results where this torch build writes them)
    if out.dtype == torch.bfloat16 or _mm_f32_out_works(out.device):
      for b in range(B):
        if out.dtype == torch.bfloat16:
          torch.mm(x[:, b * K:(b + 1) * K], w[b].t(), out=out[b])
        else:
          torch.mm(x[:, b * K:(b + 1) * K], w[b].t(), out_dtype=torch.float32, out=out[b])
      return
  linear_batched(out.transpose(0, 1), x.view(M, B, K), w)


def causal_conv(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
                ctx, silu: bool = True, in_bias: Optional[torch.Tensor] = None) -> None:
  """Short causal convolution over time per channel with the activation behind it, continuing from and updating the
  per-request state: ``out[t, c] = act(bias[c] + sum_k weight[c, taps - 1 - k] * x[t - k, c])``.  ``x`` and ``out`` may be
  column ranges of wider rows; ``state [slots, >= (taps - 1) * channels]`` float32 holds each request's last taps - 1
  inputs (oldest first) and is brought up to date after the convolution (two launches).  ``in_bias [channels]`` float32 is added
  to every input ``x[t, c]`` (the bias of the projection that made ``x``; what lies before a request's start stays zero)
  and the state keeps the inputs with it."""
  lib = common_lib()
  T, C = x.shape
  taps = weight.shape[1]
  if (weight.shape != (C, taps) or out.shape != (T, C) or out.dtype != x.dtype or (bias is not None and bias.shape != (C,))
      or (in_bias is not None and in_bias.shape != (C,))):
    raise KernelError("causal_conv: shapes do not match")
  if state.dim() != 2 or state.stride(1) != 1 or state.dtype != torch.float32:
    raise KernelError("causal_conv: the state must be float32 rows, one per request slot")
  xp, ldx = _cols(x, "causal_conv")
  op, ldo = _cols(out, "causal_conv")
  _check(lib, lib.mi_causal_conv(op, ldo, xp, ldx, _dt(x), _ptr(weight, torch.float32), _ptr(bias, torch.float32) if bias is not None else _ptr(None),
                                 _ptr(in_bias, torch.float32) if in_bias is not None else _ptr(None), ctypes.c_void_p(state.data_ptr()), ctypes.c_longlong(state.stride(0)), _ptr(ctx.token_item, torch.int32),
                                 _ptr(ctx.q_start, torch.int32), _ptr(ctx.q_len, torch.int32), _ptr(ctx.seq_slot, torch.int32),
                                 T, ctx.num_items, C, taps, int(bool(silu)), _stream()), kernels=2 if taps > 1 else 1)


SCAN_SEGMENTED_MIN_TOKENS = 512    # new tokens a request, on average, from which a bfloat16 scan runs in stretches side by side
SCAN_SEGMENTED_MAX_ITEMS = 8       # ... in steps of at most this many requests (the scratch grows with them)
DELTA_SEGMENTED_MAX_ITEMS = 4      # the same bound for the delta rule, whose scratch holds a state and a map a stretch and head
# ... and only while the walk in order would leave most SMs idle: stretches cost three times the arithmetic.  Measured on
# B200, 2048 tokens of one request, heads of 128 x 128: 8 heads (64 blocks in order) 5.18 -> 4.57 ms a step of six layers,
# 16 heads (128 blocks) 7.23 -> 8.11 ms
DELTA_SEGMENTED_MAX_BLOCKS = 96


def selective_scan(y: torch.Tensor, u: torch.Tensor, dt_in: torch.Tensor, bc: torch.Tensor, b_off: int, c_off: int, z: torch.Tensor,
                   dt_bias: torch.Tensor, A_log: torch.Tensor, D: torch.Tensor, state: torch.Tensor, ctx, workspace=None) -> None:
  """The selective scan over each item's new tokens, from and to the per-request state ``[slots, >= inner * N]`` float32:
  ``dt = softplus(dt_in + dt_bias)``, ``S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c u_c B_n`` with ``A = -exp(A_log)``,
  ``y_c = (sum_n S[c, n] C_n + D_c u_c) * silu(z_c)``; B and C are ``N`` columns of ``bc`` from ``b_off`` / ``c_off``.
  A bfloat16 step that brings long prompt portions (at least ``SCAN_SEGMENTED_MIN_TOKENS`` a request on average, few
  requests) runs each request's tokens in up to 16 stretches side by side - every stretch from a zero state, the stretches
  chained, every stretch again from the state it starts from (three launches, scratch from ``workspace``); a float32 step
  walks the tokens in order, so that its sums do not depend on how a request was cut."""
  lib = common_lib()
  T, inner = u.shape
  N = A_log.shape[1]
  if A_log.shape != (inner, N) or dt_bias.shape != (inner,) or D.shape != (inner,) or y.shape != (T, inner) or dt_in.shape != (T, inner) or z.shape != (T, inner):
    raise KernelError("selective_scan: shapes do not match")
  if bc.shape[0] != T or max(b_off, c_off) + N > bc.shape[1] or len({y.dtype, u.dtype, dt_in.dtype, bc.dtype, z.dtype}) != 1:
    raise KernelError("selective_scan: the B / C rows do not match, or the activations differ in dtype")
  if state.dim() != 2 or state.stride(1) != 1 or state.dtype != torch.float32:
    raise KernelError("selective_scan: the state must be float32 rows, one per request slot")
  (yp, ldy), (up, ldu), (dp, ldd), (bp, ldb), (zp, ldz) = (_cols(t, "selective_scan") for t in (y, u, dt_in, bc, z))
  segments, launches = None, 1
  if (u.dtype == torch.bfloat16 and ctx.num_items <= SCAN_SEGMENTED_MAX_ITEMS and T >= SCAN_SEGMENTED_MIN_TOKENS * ctx.num_items
      and os.environ.get("MINIINFER_B200_SCAN_SEGMENTS", "1") != "0"):
    n = ctx.num_items * int(lib.mi_selective_scan_segments()) * inner * (N + 1)
    segments = workspace.buffer("selective_scan_segments", (n,), torch.float32) if workspace is not None else \
      torch.empty(n, dtype=torch.float32, device=u.device)
    launches = 3
  _check(lib, lib.mi_selective_scan(yp, ldy, up, ldu, dp, ldd, bp, ldb, b_off, c_off, zp, ldz, _dt(u), _ptr(dt_bias, torch.float32),
                                    _ptr(A_log, torch.float32), _ptr(D, torch.float32), ctypes.c_void_p(state.data_ptr()),
                                    ctypes.c_longlong(state.stride(0)), _ptr(ctx.q_start, torch.int32), _ptr(ctx.q_len, torch.int32),
                                    _ptr(ctx.seq_slot, torch.int32), ctx.num_items, inner, N,
                                    _ptr(segments, torch.float32) if segments is not None else _ptr(None), _stream()), kernels=launches)


def gated_delta(out: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor, b: torch.Tensor, gate: torch.Tensor,
                dt_bias: torch.Tensor, A_log: torch.Tensor, norm_w: torch.Tensor, eps: float, state: torch.Tensor, ctx,
                heads: int, kv_heads: int, dim: int, vdim: int, workspace=None) -> None:
  """The gated delta rule over each item's new tokens, from and to the per-request state ``[slots, >= heads * dim * vdim]``
  float32.  ``q``, ``k`` ``[T, kv_heads * dim]`` (convolved and activated; made unit vectors here, q also times dim^-1/2),
  ``v [T, heads * vdim]``, ``a [T, heads * dim]`` (decay input: g = exp(-exp(A_log_h) softplus(a + dt_bias))), ``b [T, heads]``
  (beta = sigmoid(b)), ``gate [T, heads * vdim]``; per head ``S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q``;
  ``out = o / rms(o) * norm_w * sigmoid(gate)``.  All operands may be column ranges of wider rows.  Three launches: what
  does not depend on the state for all tokens at once, the recurrence, the read-outs' norm and gate; float32 scratch
  between them from ``workspace`` (a ``Workspace``; made here if absent).  A bfloat16 step of long prompt portions walks
  each request's tokens in stretches side by side (``csrc/recurrent.cu``); a float32 step walks them in order, so that its
  sums do not depend on how a request was cut."""
  lib = common_lib()
  T = v.shape[0]
  if (q.shape != (T, kv_heads * dim) or k.shape != q.shape or v.shape != (T, heads * vdim) or a.shape != (T, heads * dim) or b.shape != (T, heads)
      or gate.shape != v.shape or out.shape != v.shape or dt_bias.shape != (heads * dim,) or A_log.shape != (heads,) or norm_w.shape != (vdim,)):
    raise KernelError("gated_delta: shapes do not match")
  if len({t.dtype for t in (out, q, k, v, a, b, gate)}) != 1:
    raise KernelError("gated_delta: the activations differ in dtype")
  if state.dim() != 2 or state.stride(1) != 1 or state.dtype != torch.float32:
    raise KernelError("gated_delta: the state must be float32 rows, one per request slot")
  (op, ldo), (qp, ldq), (kp, ldk), (vp, ldv), (ap, lda), (bp, ldb), (gp, ldg) = (_cols(t, "gated_delta") for t in (out, q, k, v, a, b, gate))
  if ldq != ldk:
    raise KernelError("gated_delta: q and k must be column ranges of rows of one width")
  lib.mi_gated_delta_scratch_floats.restype = ctypes.c_longlong
  n = int(lib.mi_gated_delta_scratch_floats(T, heads, kv_heads, dim, vdim)) + 8
  scratch = workspace.buffer("gated_delta_scratch", (n,), torch.float32) if workspace is not None else \
    torch.empty(n, dtype=torch.float32, device=v.device)
  # long prompt portions in bfloat16: each request's tokens in up to 16 stretches side by side (five launches instead of three)
  segments, launches = None, 3
  if (v.dtype == torch.bfloat16 and ctx.num_items <= DELTA_SEGMENTED_MAX_ITEMS and T >= SCAN_SEGMENTED_MIN_TOKENS * ctx.num_items
      and dim <= 256 and ctx.num_items * int(lib.mi_gated_delta_blocks(heads, dim, vdim)) <= DELTA_SEGMENTED_MAX_BLOCKS
      and os.environ.get("MINIINFER_B200_DELTA_SEGMENTS", "1") != "0"):
    m = ctx.num_items * int(lib.mi_gated_delta_segments()) * heads * dim * (vdim + dim)
    segments = workspace.buffer("gated_delta_segments", (m,), torch.float32) if workspace is not None else \
      torch.empty(m, dtype=torch.float32, device=v.device)
    launches = 5
  _check(lib, lib.mi_gated_delta(op, ldo, qp, kp, ldq, vp, ldv, ap, lda, bp, ldb, gp, ldg, _dt(v), _ptr(dt_bias, torch.float32),
                                 _ptr(A_log, torch.float32), _ptr(norm_w, torch.float32), ctypes.c_float(eps),
                                 ctypes.c_void_p(state.data_ptr()), ctypes.c_longlong(state.stride(0)), _ptr(ctx.q_start, torch.int32),
                                 _ptr(ctx.q_len, torch.int32), _ptr(ctx.seq_slot, torch.int32), T, ctx.num_items, heads, kv_heads, dim, vdim,
                                 _ptr(scratch, torch.float32), _ptr(segments, torch.float32) if segments is not None else _ptr(None),
                                 _stream()), kernels=launches)


LINEAR_SEGMENTED_MAX_ITEMS = 8     # steps of at most this many requests run long bfloat16 portions in stretches side by side
# ... and only while the walk in order would leave SMs idle (blocks in order, all requests; an SM holds three, and
# stretches cost twice the arithmetic).  Measured on B200, 8192 tokens of one request beside seven single tokens, 16 heads
# of 128 x 128 (8 x 32 blocks in order): 4.7 ms in order.
LINEAR_SEGMENTED_MAX_BLOCKS = 256


def linear_attention(out: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gate: torch.Tensor, state: torch.Tensor, ctx,
                     heads: int, dim: int, vdim: int, eps: float, decay_logits: Optional[torch.Tensor] = None,
                     decay_bias: Optional[torch.Tensor] = None, tau: float = 1.0, head_decay: Optional[torch.Tensor] = None,
                     rope: Optional[torch.Tensor] = None, q_scale: float = 1.0, k_scale: float = 1.0,
                     norm_weight: Optional[torch.Tensor] = None, gate_silu: bool = True, workspace=None) -> None:
  """Linear attention with a decaying state over each item's new tokens, from and to the per-request state
  ``[slots, >= heads * dim * vdim]`` float32: per head ``S <- diag(alpha) S + k v^T; o = S^T q`` with
  ``alpha = exp(logsigmoid(decay_logits + decay_bias) / tau)`` per token and key channel (``decay_logits [T, heads * dim]``
  float32) or the constant ``head_decay[h]`` (float32 ``[heads]``); ``out = o / rms(o) * norm_weight * act(gate)``, ``act`` =
  silu or sigmoid, ``norm_weight [vdim]`` optional.  ``q``, ``k`` ``[T, heads * dim]`` are first rotated by the token's position
  (``rope [positions, rot_dims]``, cos then sin; value i with value i + rot_dims / 2) and scaled.  ``q``, ``k``, ``v``, ``gate``
  and ``out`` may be column ranges of wider rows.  Three launches; a bfloat16 step of long prompt portions walks each
  request's tokens in stretches side by side (five launches), a float32 step always in order."""
  lib = common_lib()
  T = v.shape[0]
  if (q.shape != (T, heads * dim) or k.shape != q.shape or v.shape != (T, heads * vdim) or gate.shape != v.shape or out.shape != v.shape
      or (norm_weight is not None and norm_weight.shape != (vdim,))):
    raise KernelError("linear_attention: shapes do not match")
  if len({t.dtype for t in (out, q, k, v, gate)}) != 1:
    raise KernelError("linear_attention: the activations differ in dtype")
  if (decay_logits is None) == (head_decay is None):
    raise KernelError("linear_attention: give the decays' logits or the heads' constants, one of the two")
  if decay_logits is not None and (decay_logits.shape != (T, heads * dim) or decay_logits.dtype != torch.float32
                                   or (decay_bias is not None and decay_bias.shape != (heads * dim,))):
    raise KernelError("linear_attention: the decays' logits must be float32 [tokens, heads * dim], their bias [heads * dim]")
  if head_decay is not None and head_decay.shape != (heads,):
    raise KernelError("linear_attention: one constant decay a head")
  if state.dim() != 2 or state.stride(1) != 1 or state.dtype != torch.float32:
    raise KernelError("linear_attention: the state must be float32 rows, one per request slot")
  (op, ldo), (qp, ldq), (kp, ldk), (vp, ldv), (gp, ldg) = (_cols(t, "linear_attention") for t in (out, q, k, v, gate))
  ap, lda = _cols(decay_logits, "linear_attention") if decay_logits is not None else (_ptr(None), 0)
  channel = decay_logits is not None
  lib.mi_linear_attention_scratch_floats.restype = ctypes.c_longlong
  n = int(lib.mi_linear_attention_scratch_floats(T, heads, dim, vdim, int(channel))) + 8
  scratch = workspace.buffer("linear_attention_scratch", (n,), torch.float32) if workspace is not None else \
    torch.empty(n, dtype=torch.float32, device=v.device)
  segments, launches = None, 3
  if (v.dtype == torch.bfloat16 and ctx.num_items <= LINEAR_SEGMENTED_MAX_ITEMS and T >= SCAN_SEGMENTED_MIN_TOKENS * ctx.num_items
      and ctx.num_items * int(lib.mi_linear_attention_blocks(heads, dim, vdim)) <= LINEAR_SEGMENTED_MAX_BLOCKS
      and os.environ.get("MINIINFER_B200_LINEAR_SEGMENTS", "1") != "0"):
    m = ctx.num_items * int(lib.mi_linear_attention_segments()) * heads * dim * (vdim + 1)
    segments = workspace.buffer("linear_attention_segments", (m,), torch.float32) if workspace is not None else \
      torch.empty(m, dtype=torch.float32, device=v.device)
    launches = 5
  none = _ptr(None)
  _check(lib, lib.mi_linear_attention(
    op, ldo, qp, ldq, kp, ldk, vp, ldv, gp, ldg, _dt(v), ap, lda,
    _ptr(decay_bias, torch.float32) if (channel and decay_bias is not None) else none, ctypes.c_float(1.0 / tau),
    _ptr(head_decay, torch.float32) if head_decay is not None else none,
    _ptr(rope, torch.float32) if rope is not None else none, _ptr(ctx.positions, torch.int32) if rope is not None else none,
    int(rope.shape[1]) if rope is not None else 0, ctypes.c_float(q_scale), ctypes.c_float(k_scale),
    _ptr(norm_weight, torch.float32) if norm_weight is not None else none, ctypes.c_float(eps), int(bool(gate_silu)),
    ctypes.c_void_p(state.data_ptr()), ctypes.c_longlong(state.stride(0)), _ptr(ctx.q_start, torch.int32), _ptr(ctx.q_len, torch.int32),
    _ptr(ctx.seq_slot, torch.int32), T, ctx.num_items, heads, dim, vdim, _ptr(scratch, torch.float32),
    _ptr(segments, torch.float32) if segments is not None else none, _stream()), kernels=launches)


def token_shift(out: torch.Tensor, resid: torch.Tensor, shift: Optional[torch.Tensor], state: Optional[torch.Tensor], ctx) -> None:
  """out[t] = x[t] + (x[t - 1] - x[t]) * shift for the float32 rows ``x = resid``, written in ``out``'s dtype; ``x[t - 1]`` of an
  item's first new token is the item's row of ``state [slots, >= width]`` float32 (zeros for a request's first token), which is
  only read here.  Without ``shift``: a copy of the rows into ``out``'s dtype."""
  lib = common_lib()
  T, W = resid.shape
  if out.shape != (T, W) or resid.dtype != torch.float32 or not (resid.is_contiguous() and out.is_contiguous()):
    raise KernelError("token_shift: shapes do not match or rows are not contiguous")
  if shift is not None and (shift.shape != (W,) or state is None or state.dim() != 2 or state.stride(1) != 1 or state.dtype != torch.float32
                            or state.shape[1] < W):
    raise KernelError("token_shift: the shift is one float32 per channel and needs float32 state rows of the width")
  _check(lib, lib.mi_token_shift(_ptr(out), _dt(out), _ptr(resid, torch.float32), T, W,
                                 _ptr(shift, torch.float32) if shift is not None else _ptr(None),
                                 ctypes.c_void_p(state.data_ptr()) if shift is not None else _ptr(None),
                                 ctypes.c_longlong(state.stride(0) if shift is not None else 0), _ptr(ctx.token_item, torch.int32),
                                 _ptr(ctx.q_start, torch.int32), _ptr(ctx.seq_slot, torch.int32), _stream()))


def norm_scaled_add(resid: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, mult: float, ctx,
                    copy: Optional[torch.Tensor] = None, keep: Optional[torch.Tensor] = None) -> None:
  """resid[t] += mult * weight * y[t] / sqrt(mean(y[t]^2) + eps) in float32, in place: the RMS norm of a sublayer's output
  added to the residual rows.  ``copy [T, W]`` (``y``'s dtype) receives the new rows; ``keep [slots, >= W]`` float32 receives,
  for the last new token of every item, the row as it was BEFORE the addition (the state of a token shift)."""
  lib = common_lib()
  T, W = resid.shape
  if y.shape != (T, W) or weight.shape != (W,) or resid.dtype != torch.float32 or not (resid.is_contiguous() and y.is_contiguous()):
    raise KernelError("norm_scaled_add: shapes do not match or rows are not contiguous")
  if copy is not None and (copy.shape != (T, W) or copy.dtype != y.dtype or not copy.is_contiguous()):
    raise KernelError("norm_scaled_add: the copy has the rows' shape and the sublayer output's dtype")
  if keep is not None and (keep.dim() != 2 or keep.stride(1) != 1 or keep.dtype != torch.float32 or keep.shape[1] < W):
    raise KernelError("norm_scaled_add: the kept rows are float32 state rows of the width")
  _check(lib, lib.mi_norm_scaled_add(_ptr(resid, torch.float32), _ptr(y), _dt(y), _ptr(weight, torch.float32), T, W, ctypes.c_float(eps),
                                     ctypes.c_float(mult), _ptr(copy) if copy is not None else _ptr(None), _dt(y),
                                     ctypes.c_void_p(keep.data_ptr()) if keep is not None else _ptr(None),
                                     ctypes.c_longlong(keep.stride(0) if keep is not None else 0), _ptr(ctx.token_item, torch.int32),
                                     _ptr(ctx.q_start, torch.int32), _ptr(ctx.q_len, torch.int32), _ptr(ctx.seq_slot, torch.int32), _stream()))


RECURRENCE_SEGMENTED_MIN_TOKENS = 512   # new tokens a request, on average, from which a bfloat16 diagonal recurrence runs in stretches side by side
RECURRENCE_SEGMENT_MIN = 16             # ... the items of at least this many tokens a stretch


def _recurrence_segmented(dtype: torch.dtype, ctx) -> int:
  """Whether a step's diagonal recurrences take the form with stretches side by side: bfloat16 steps of long portions.  The
  choice depends on the step's counts of tokens and items only, which are part of a recorded graph's identity."""
  return int(dtype == torch.bfloat16 and ctx.num_tokens >= RECURRENCE_SEGMENTED_MIN_TOKENS * max(1, ctx.num_items)
             and os.environ.get("MINIINFER_B200_RECURRENCE_SEGMENTS", "1") != "0")


def _state_rows_arg(state: torch.Tensor, width: int, what: str):
  if state.dim() != 2 or state.stride(1) != 1 or state.dtype != torch.float32 or state.shape[1] < width:
    raise KernelError(f"{what}: the state must be float32 rows of at least {width} values, one per request slot")
  return ctypes.c_void_p(state.data_ptr()), ctypes.c_longlong(state.stride(0))


def _recurrence_scratch(workspace, segmented: int, T: int, C: int):
  """Scratch of the segmented form: what the tokens give the channels, prepared by a kernel of its own."""
  if not segmented or workspace is None:
    return 0, _ptr(None)
  return T, _ptr(workspace.buffer("recurrence_prepared", (3 * T * C,), torch.float32))


def rglru_recurrence(out: torch.Tensor, u: torch.Tensor, gates: torch.Tensor, y: torch.Tensor, r_bias: torch.Tensor, i_bias: torch.Tensor,
                     y_bias: Optional[torch.Tensor], lam: torch.Tensor, state: torch.Tensor, ctx, blocks: int, workspace=None) -> None:
  """The real-gated linear recurrent unit over the channels of ``u [T, C]``: with ``gates`` float32, ``[T, 2 C]`` (token after
  token, part after part) or ``[blocks, T, 2 C / blocks]`` (part after part, as one product a part leaves them) - a
  part's logits of r, then of i -, ``r = sigmoid(. + r_bias)``, ``i = sigmoid(. + i_bias)``, ``a = exp(-8 r softplus(lam))``,
  ``S <- a S + sqrt(1 - a^2) i u`` from the item's row of ``state``, and ``out = S * gelu_tanh(y + y_bias)``.  ``u``, ``y``, ``out``
  may be column ranges of wider rows; biases and ``lam`` are float32 ``[C]``.  ``workspace`` lends the scratch of the form
  with stretches side by side (long bfloat16 portions)."""
  lib = common_lib()
  T, C = u.shape
  if (out.shape != (T, C) or y.shape != (T, C) or gates.dtype != torch.float32 or not gates.is_contiguous()
      or out.dtype != u.dtype or y.dtype != u.dtype or C % blocks or tuple(gates.shape) not in ((T, 2 * C), (blocks, T, 2 * C // blocks))):
    raise KernelError("rglru_recurrence: shapes or dtypes do not match")
  by_part = gates.dim() == 3
  ldg, part_stride = (2 * C // blocks, T * 2 * C // blocks) if by_part else (2 * C, 2 * C // blocks)
  for b in (r_bias, i_bias, lam) + ((y_bias,) if y_bias is not None else ()):
    if b.shape != (C,) or b.dtype != torch.float32:
      raise KernelError("rglru_recurrence: biases and lam are one float32 per channel")
  (op, ldo), (up, ldu), (yp, ldy) = _cols(out, "rglru_recurrence"), _cols(u, "rglru_recurrence"), _cols(y, "rglru_recurrence")
  sp, ss = _state_rows_arg(state, C, "rglru_recurrence")
  segmented = _recurrence_segmented(u.dtype, ctx)
  rows, scratch = _recurrence_scratch(workspace, segmented, T, C)
  _check(lib, lib.mi_rglru_recurrence(op, ldo, up, ldu, _ptr(gates, torch.float32), ldg, ctypes.c_longlong(part_stride), yp, ldy, _dt(u),
                                      _ptr(r_bias, torch.float32),
                                      _ptr(i_bias, torch.float32), _ptr(y_bias, torch.float32) if y_bias is not None else _ptr(None),
                                      _ptr(lam, torch.float32), sp, ss, _ptr(ctx.q_start, torch.int32), _ptr(ctx.q_len, torch.int32),
                                      _ptr(ctx.seq_slot, torch.int32), ctx.num_items, C, blocks, segmented,
                                      RECURRENCE_SEGMENT_MIN, rows, scratch, _stream()), kernels=2 if rows else 1)


def mingru_recurrence(out: torch.Tensor, proj: torch.Tensor, z_bias: Optional[torch.Tensor], x_bias: Optional[torch.Tensor],
                      state: torch.Tensor, ctx, workspace=None) -> None:
  """The minimal gated recurrence over ``proj [T, 3 C]`` (logits of z, then x, then g): ``z = sigmoid(. + z_bias)``, the candidate
  ``c = x + 1/2`` where ``x = . + x_bias >= 0`` and ``sigmoid(x)`` below, ``S <- (1 - z) S + z c`` from the item's row of ``state``,
  ``out = S * silu(g)``."""
  lib = common_lib()
  T, C = out.shape
  if proj.shape != (T, 3 * C) or proj.dtype != out.dtype:
    raise KernelError("mingru_recurrence: shapes or dtypes do not match")
  for b in (z_bias, x_bias):
    if b is not None and (b.shape != (C,) or b.dtype != torch.float32):
      raise KernelError("mingru_recurrence: biases are one float32 per channel")
  (op, ldo), (pp, ld) = _cols(out, "mingru_recurrence"), _cols(proj, "mingru_recurrence")
  sp, ss = _state_rows_arg(state, C, "mingru_recurrence")
  segmented = _recurrence_segmented(out.dtype, ctx)
  rows, scratch = _recurrence_scratch(workspace, segmented, T, C)
  _check(lib, lib.mi_mingru_recurrence(op, ldo, pp, ld, _dt(out), _ptr(z_bias, torch.float32) if z_bias is not None else _ptr(None),
                                       _ptr(x_bias, torch.float32) if x_bias is not None else _ptr(None), sp, ss,
                                       _ptr(ctx.q_start, torch.int32), _ptr(ctx.q_len, torch.int32), _ptr(ctx.seq_slot, torch.int32),
                                       ctx.num_items, C, segmented, RECURRENCE_SEGMENT_MIN, rows, scratch, _stream()),
         kernels=2 if rows else 1)


def hyper_connection(res: torch.Tensor, streams: torch.Tensor, y: Optional[torch.Tensor], mix: Optional[torch.Tensor],
                     out_w: Optional[torch.Tensor], in_w: Optional[torch.Tensor], norm_weight: Optional[torch.Tensor], eps: float,
                     rows: Optional[torch.Tensor] = None, write_back: bool = True) -> None:
  """One pass over residual streams ``[tokens, S * width]`` float32 (stream after stream in a row).  With ``y [tokens, width]``
  the streams are first brought up to date, all at once from the old ones: ``x_t <- sum_s mix[s, t] x_s + out_w[t] y`` (written
  back if ``write_back``).  Then ``u = sum_t in_w[t] x_t`` (``in_w`` None: the plain sum) and ``res = norm_weight * u / sqrt(mean(u^2)
  + eps)``, or ``res = u`` without ``norm_weight``.  ``rows`` selects rows of the streams (``res`` has one row per selected row).
  All float32; ``res`` is rounded once to its dtype."""
  lib = common_lib()
  R, W = res.shape
  if streams.dim() != 2 or streams.shape[1] % W or streams.dtype != torch.float32:
    raise KernelError("hyper_connection: the streams must be float32 rows of a whole number of streams")
  S = streams.shape[1] // W
  if (rows is None and streams.shape[0] != R) or (rows is not None and rows.shape[0] != R):
    raise KernelError("hyper_connection: res, rows and the streams differ in rows")
  if y is not None and (y.shape != (streams.shape[0], W) or mix is None or out_w is None or mix.shape != (S, S) or out_w.shape != (S,)):
    raise KernelError("hyper_connection: an update needs y [tokens, width], mix [S, S] and out [S]")
  if (in_w is not None and in_w.shape != (S,)) or (norm_weight is not None and norm_weight.shape != (W,)):
    raise KernelError("hyper_connection: the read weights do not match")
  none = _ptr(None)
  _check(lib, lib.mi_hyper_connection(
    _ptr(res), _dt(res), _ptr(streams, torch.float32), _ptr(y) if y is not None else none, _dt(y) if y is not None else F32,
    _ptr(mix, torch.float32) if y is not None else none, _ptr(out_w, torch.float32) if y is not None else none,
    _ptr(in_w, torch.float32) if in_w is not None else none, _ptr(norm_weight, torch.float32) if norm_weight is not None else none,
    _ptr(rows, torch.int32) if rows is not None else none, R, S, W, ctypes.c_float(eps), int(bool(write_back)), _stream()))


def relu_squared(out: torch.Tensor, x: torch.Tensor) -> None:
  """out = max(x, 0)^2 element by element, squared in float32 and rounded once; ``out`` may be ``x``."""
  lib = common_lib()
  if out.shape != x.shape or out.dtype != x.dtype:
    raise KernelError("relu_squared: out and x differ")
  _check(lib, lib.mi_relu_squared(_ptr(out), _ptr(x), _dt(x), ctypes.c_longlong(x.numel()), _stream()))


def linear_relu_squared(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, workspace, force_tc: bool = False) -> None:
  """out[M, N] = max(x @ w^T, 0)^2: the up product of a squared-ReLU feed-forward.  bfloat16 with M <= 16 (below the
  sizes of the weight-streaming tcgen05 kernel) or from 1280 rows on (1792 for K < 4096): one kernel, the activation in
  the product's epilogue (few rows: the mma.sync kernel; many: the tcgen05 kernel) - the product is rounded to bfloat16
  before it is clamped and squared, so the values are those of the product followed by the activation kernel, which is
  what runs otherwise (``MINIINFER_B200_RELU2_FUSED=0``: always)."""
  M, K = x.shape
  N = w.shape[0]
  if w.shape[1] != K or out.shape != (M, N) or out.dtype != x.dtype:
    raise KernelError(f"linear_relu_squared: shapes do not match: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
  if M == 0:
    return
  fits = (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K >= 64 and K % 8 == 0 and N % 8 == 0 and x.is_contiguous()
          and w.is_contiguous() and out.is_contiguous() and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0
          and os.environ.get("MINIINFER_B200_RELU2_FUSED", "1") != "0")
  if fits and M <= SKINNY_BEST_M and not _streams(M, N, K, False, False):
    lib = common_lib()
    _check(lib, lib.mi_gemm_skinny_relu2_bf16(_ptr(out), _ptr(x), _ptr(w), M, N, K, N, _stream()))
    return
  many = force_tc or M >= (GEMM_TC_MIN_M if K >= 4096 else GEMM_TC_MIN_M_NARROW)
  if fits and many and os.environ.get("MINIINFER_B200_GEMM_TC", "1") != "0":
    lib = common_lib()
    status = workspace.zeros("gemm_tc_status", 1, torch.int32)
    _check(lib, lib.mi_gemm_tc_relu2_bf16(_ptr(out), _ptr(x), _ptr(w), M, N, K, N, _ptr(status, torch.int32), _tc_pairs(), _stream()))
    return
  linear(out, x, w)
  relu_squared(out, out)


def scaled_pair_sum(out: torch.Tensor, a: torch.Tensor, b: torch.Tensor, scale_a: float, scale_b: float) -> None:
  """out = scale_a * a + scale_b * b element by element, in float32, rounded once."""
  lib = common_lib()
  if a.shape != out.shape or b.shape != out.shape or a.dtype != out.dtype or b.dtype != out.dtype:
    raise KernelError("scaled_pair_sum: shapes or dtypes do not match")
  _check(lib, lib.mi_scaled_pair_sum(_ptr(out), _ptr(a), _ptr(b), _dt(out), ctypes.c_longlong(out.numel()),
                                     ctypes.c_float(scale_a), ctypes.c_float(scale_b), _stream()))


def latent_down(down: torch.Tensor, q_off: int, kv_off: int, q_rank: int, kv_rank: int, rot_dim: int, q_weight: torch.Tensor,
                kv_weight: torch.Tensor, eps: float, cq_out: torch.Tensor, rope: torch.Tensor, positions: torch.Tensor, interleaved: bool,
                slot_mapping: Optional[torch.Tensor], kv_layer: Optional[torch.Tensor]) -> None:
  """From the fused down-projection rows of a latent attention: the RMS-normed query latent (``q_rank`` values at ``q_off``)
  into ``cq_out [T, q_rank]``; the RMS-normed key/value latent (``kv_rank`` values at ``kv_off``) and the rotated shared key
  part (``rot_dim`` values behind it) into the layer's pages: key row ``[c | k_rot | 0]``, value row ``[c | 0]``."""
  lib = common_lib()
  T = down.shape[0]
  if max(q_off + q_rank, kv_off + kv_rank + rot_dim) > down.shape[1] or cq_out.shape != (T, q_rank) or cq_out.dtype != down.dtype:
    raise KernelError("latent_down: the latents do not fit the projection rows")
  if rope.shape[1] != rot_dim or q_weight.shape != (q_rank,) or kv_weight.shape != (kv_rank,):
    raise KernelError("latent_down: weights or rotation table do not match")
  hdp, page_size = kv_rank + rot_dim, 0
  if kv_layer is not None:
    if kv_layer.dtype != down.dtype or kv_layer.dim() != 5 or kv_layer.shape[1:3] != (2, 1) or kv_layer.shape[4] < kv_rank + rot_dim:
      raise KernelError(f"latent_down: cache layer has shape {tuple(kv_layer.shape)}")
    page_size, hdp = kv_layer.shape[3], kv_layer.shape[4]
  none = _ptr(None)
  _check(lib, lib.mi_latent_down(_ptr(down), _dt(down), down.shape[1], q_off, kv_off, T, q_rank, kv_rank, rot_dim, hdp,
                                 _ptr(q_weight, torch.float32), _ptr(kv_weight, torch.float32), ctypes.c_float(eps), _ptr(cq_out),
                                 _ptr(rope, torch.float32), _ptr(positions, torch.int32), int(bool(interleaved)),
                                 _ptr(slot_mapping, torch.int32) if (slot_mapping is not None and kv_layer is not None) else none,
                                 _ptr(kv_layer) if kv_layer is not None else none, page_size, _stream()))


def latent_query(q: torch.Tensor, q_out: torch.Tensor, heads: int, dim: int, rot_dim: int, kv_rank: int, rope: torch.Tensor,
                 positions: torch.Tensor, interleaved: bool) -> None:
  """The rotated part of every query head (``rot_dim`` values behind the head's ``dim`` unrotated ones in ``q [T, heads * (dim +
  rot_dim)]``), rotated, into ``q_out [T, heads * hdp]`` behind each head's first ``kv_rank`` values; the rest of a head is zeroed."""
  lib = common_lib()
  T = q.shape[0]
  hdp = q_out.shape[1] // heads
  if q.shape != (T, heads * (dim + rot_dim)) or q_out.shape != (T, heads * hdp) or hdp < kv_rank + rot_dim or q_out.dtype != q.dtype or rope.shape[1] != rot_dim:
    raise KernelError("latent_query: shapes do not match")
  _check(lib, lib.mi_latent_query(_ptr(q), _dt(q), q.shape[1], T, heads, dim, rot_dim, kv_rank, hdp, _ptr(q_out), _ptr(rope, torch.float32),
                                  _ptr(positions, torch.int32), int(bool(interleaved)), _stream()))


MOE_TC_ROW_TILE = 256            # rows of a stretch of the tcgen05 grouped product: what a pair of blocks takes at a time
MOE_TC_MIN_ROWS_PER_EXPERT = 128   # from this many (token, choice) pairs per expert on, on average, the tcgen05 product runs


def moe_row_tile(num_pairs: int, num_experts: int, dtype: torch.dtype) -> int:
  """Rows of a row tile of the grouped products for a step with ``num_pairs`` (token, choice) pairs."""
  return int(common_lib().mi_moe_row_tile(num_pairs, num_experts, F32 if dtype == torch.float32 else BF16))


def moe_rows(num_pairs: int, num_experts: int, tile: int) -> int:
  """Rows that hold ``num_pairs`` pairs when every expert's rows start at a multiple of ``tile``, in the worst case."""
  return -(-(num_pairs + num_experts * (tile - 1)) // tile) * tile


GLU_KINDS = {"silu": 0, "clamped": 1}      # the gated activations of common.cuh (MiGlu)


def _glu(kind: str, limit: float):
  if kind not in GLU_KINDS or (kind == "clamped" and not limit > 0):
    raise KernelError(f"gated activation {kind!r} is not known ({', '.join(GLU_KINDS)}) or its limit {limit!r} is not positive")
  return GLU_KINDS[kind], ctypes.c_float(float(limit))


def routed_experts(out: torch.Tensor, x: torch.Tensor, router: torch.Tensor, correction: Optional[torch.Tensor], gate_up: torch.Tensor,
                   down: torch.Tensor, top: int, workspace, weights: str = "sigmoid_share", glu: str = "silu", limit: float = 0.0,
                   shared: Optional[torch.Tensor] = None, shared_gated: bool = False) -> None:
  """out[t] = sum over the ``top`` chosen experts of weight * down_e(silu(gate_e x) * up_e x).

  ``router [E, H]`` in the rows' dtype and ``correction [E]`` float32: logits ``router x`` accumulated in float32 (bfloat16
  operands multiply exactly in float32), scores their sigmoid; the ``top`` experts of largest
  score + correction are chosen; weights are their scores divided by the scores' sum (+ 1e-20).  ``gate_up [E, 2 ff, H]``
  (an expert's gate rows, then its up rows) and ``down [E, H, ff]`` in the rows' dtype.  Six or seven launches, nothing read
  back by the host; scratch from ``workspace``.

  ``weights="softmax_chosen"``: the ``top`` largest logits are chosen (``correction`` may be None) and the weights are the
  softmax over the chosen logits alone.  ``glu``/``limit``: the experts' gated activation (``silu``, or ``clamped`` with its
  limit: ``g' = min(g, L)``, ``u' = clamp(u, -L, L)``, ``g' sigmoid(1.702 g') (u' + 1)``).  ``shared [T, H]``: the output of an
  expert that every token runs through, added to the sum; with ``shared_gated`` the router has one row more than there are
  experts, and the shared rows are multiplied with the sigmoid of that row's logit, one number a token."""
  lib = common_lib()
  T, H = x.shape
  E = router.shape[0] - (1 if shared_gated else 0)
  ff = down.shape[2]
  if weights not in ("sigmoid_share", "softmax_chosen") or (correction is None and weights == "sigmoid_share"):
    raise KernelError(f"routed_experts: weights={weights!r} is not known, or sigmoid shares without their correction")
  if shared_gated and shared is None:
    raise KernelError("routed_experts: a gate for the shared expert without its rows")
  if shared is not None and (shared.shape != (T, H) or shared.dtype != out.dtype or not shared.is_contiguous()):
    raise KernelError("routed_experts: the shared expert's rows do not match the output")
  kind, lim = _glu(glu, limit)
  if router.shape != (E + (1 if shared_gated else 0), H) or (correction is not None and correction.shape != (E,)) or gate_up.shape != (E, 2 * ff, H) or down.shape != (E, H, ff) or out.shape != (T, H):
    raise KernelError(f"routed_experts: shapes do not match: x {tuple(x.shape)}, router {tuple(router.shape)}, "
                      f"gate_up {tuple(gate_up.shape)}, down {tuple(down.shape)}")
  if gate_up.dtype != x.dtype or down.dtype != x.dtype or out.dtype != x.dtype or router.dtype != x.dtype:
    raise KernelError("routed_experts: rows, experts and out must share a dtype")
  if T == 0:
    return
  pairs = T * top
  # Many rows per expert in bfloat16: the products on tcgen05 (gemm_tc.cu in its grouped form) over rows gathered into the
  # experts' order, every expert's rows starting at a multiple of 256.  Otherwise the mma.sync / FMA kernels of moe.cu,
  # which gather as they load and take row tiles of 16 or 64.
  on_tc = (x.dtype == torch.bfloat16 and pairs >= MOE_TC_MIN_ROWS_PER_EXPERT * E and H >= 64 and ff >= 64 and H % 8 == 0 and ff % 8 == 0
           and os.environ.get("MINIINFER_B200_MOE_TC", "1") != "0")
  tile = MOE_TC_ROW_TILE if on_tc else moe_row_tile(pairs, E, x.dtype)
  rows = moe_rows(pairs, E, tile)
  tiles = rows // tile
  idx = workspace.buffer("moe_choice", (pairs,), torch.int32)
  wts = workspace.buffer("moe_weight", (pairs,), torch.float32)
  sorted_pair = workspace.buffer("moe_sorted", (rows,), torch.int32)
  pos_of = workspace.buffer("moe_pos", (pairs,), torch.int32)
  tile_expert = workspace.buffer("moe_tile_expert", (tiles,), torch.int32)
  act = workspace.buffer("moe_act", (rows, ff), x.dtype)
  y = None if on_tc else workspace.buffer("moe_y", (rows, H), torch.float32)
  dt, st = _dt(x), _stream()
  Z = router.shape[0]
  logits = workspace.buffer("moe_logits", (T, Z), torch.float32)
  linear(logits, x, router)
  _check(lib, lib.mi_moe_route(_ptr(logits, torch.float32), Z, T, _ptr(correction, torch.float32) if correction is not None else _ptr(None), E, top,
                               1 if weights == "softmax_chosen" else 0, _ptr(idx), _ptr(wts), st))
  shared_args = (_ptr(shared) if shared is not None else _ptr(None),
                 ctypes.c_void_p(logits.data_ptr() + 4 * E) if shared_gated else _ptr(None), Z)
  _check(lib, lib.mi_moe_align(_ptr(idx), pairs, E, tile, _ptr(sorted_pair), _ptr(pos_of), _ptr(tile_expert), rows, tiles, st))
  if on_tc:
    xs = workspace.buffer("moe_rows", (rows, H), x.dtype)
    y16 = workspace.buffer("moe_y16", (rows, H), x.dtype)
    status = workspace.zeros("gemm_tc_status", 1, torch.int32)
    _check(lib, lib.mi_moe_gather(_ptr(xs), _ptr(x), _ptr(sorted_pair), rows, top, H, st))
    _check(lib, lib.mi_gemm_tc_grouped_bf16(_ptr(act), _ptr(xs), _ptr(gate_up), rows, ff, H, ff, E, 1, _ptr(tile_expert), tile,
                                            _ptr(status, torch.int32), _tc_pairs(), kind, lim, st))
    _check(lib, lib.mi_gemm_tc_grouped_bf16(_ptr(y16), _ptr(act), _ptr(down), rows, H, ff, H, E, 0, _ptr(tile_expert), tile,
                                            _ptr(status, torch.int32), _tc_pairs(), 0, ctypes.c_float(0.0), st))
    _check(lib, lib.mi_moe_combine(_ptr(out), _dt(out), _ptr(y16), BF16, _ptr(pos_of), _ptr(wts), T, top, H, *shared_args, st))
    return
  _check(lib, lib.mi_moe_gemm(_ptr(x), dt, H, _ptr(gate_up), _ptr(act), _ptr(sorted_pair), _ptr(tile_expert), tiles, tile, ff, H, top, 1, kind, lim, st))
  _check(lib, lib.mi_moe_gemm(_ptr(act), dt, ff, _ptr(down), _ptr(y), _ptr(sorted_pair), _ptr(tile_expert), tiles, tile, H, ff, top, 0, 0,
                              ctypes.c_float(0.0), st))
  _check(lib, lib.mi_moe_combine(_ptr(out), _dt(out), _ptr(y), F32, _ptr(pos_of), _ptr(wts), T, top, H, *shared_args, st))


def linear_swiglu(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, workspace, force_skinny: bool = False,
                  force_tc: bool = False, force_stream: bool = False) -> None:
  """out[M, I] = silu(x @ w[:I]^T) * (x @ w[I:]^T): the gate-and-up product of a SwiGLU feed-forward.
  bfloat16 with M <= 16 or from 1280 rows on (1792 for K < 4096): one kernel, the activation in the product's
  epilogue (few rows: the weight-streaming kernel; many: the tcgen05 kernel).  Otherwise the product into a buffer of
  ``workspace``, then the activation kernel (the same up to the order of the sums over K)."""
  M, K = x.shape
  I = out.shape[1]
  if w.shape != (2 * I, K) or out.shape[0] != M or out.dtype != x.dtype:
    raise KernelError(f"linear_swiglu: shapes do not match: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
  if M == 0:
    return
  if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and _streams(M, 2 * I, K, force_skinny, force_stream):
    lib = common_lib()
    parts, counters, status = _stream_workspace(lib, x.device)
    _check(lib, lib.mi_gemm_stream_tc_swiglu_bf16(_ptr(out), _ptr(x), _ptr(w), M, I, K, I, _ptr(parts, torch.float32),
                                                  _ptr(counters, torch.int32), counters.numel(), parts.shape[0],
                                                  _ptr(status, torch.int32), _stream()))
    return
  if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and (M <= SKINNY_BEST_M or (force_skinny and M <= SKINNY_MAX_M)):
    lib = common_lib()
    _check(lib, lib.mi_gemm_skinny_swiglu_bf16(_ptr(out), _ptr(x), _ptr(w), M, I, K, I, _stream()))
    return
  many = force_tc or M >= (GEMM_TC_MIN_M if K >= 4096 else GEMM_TC_MIN_M_NARROW)
  if (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and many and K >= 64 and K % 8 == 0 and I % 8 == 0
      and x.is_contiguous() and w.is_contiguous() and out.is_contiguous() and os.environ.get("MINIINFER_B200_GEMM_TC", "1") != "0"):
    # many rows: the product on tcgen05 with the activation in its epilogue; [M, 2I] is never written
    lib = common_lib()
    status = workspace.zeros("gemm_tc_status", 1, torch.int32)
    _check(lib, lib.mi_gemm_tc_swiglu_bf16(_ptr(out), _ptr(x), _ptr(w), M, I, K, I, _ptr(status, torch.int32), _tc_pairs(), _stream()))
    return
  gu = workspace.buffer("gate_up", (M, 2 * I), x.dtype)
  linear(gu, x, w)
  silu_mul(out, gu)


def _tc_pairs() -> int:
  """Whether the tcgen05 product lets two blocks share a tile (MINIINFER_B200_GEMM_TC=1: blocks work alone)."""
  return 0 if os.environ.get("MINIINFER_B200_GEMM_TC", "2") == "1" else 1


def linear_tc(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, workspace) -> None:
  """out = x @ w^T in bfloat16 through the tcgen05 kernel that `linear_swiglu` uses for many rows,
  without the activation (the engine's plain products with many rows go to the library)."""
  M, K = x.shape
  N = w.shape[0]
  if w.shape[1] != K or out.shape != (M, N) or not (x.dtype == w.dtype == out.dtype == torch.bfloat16):
    raise KernelError(f"linear_tc: shapes or dtypes do not match: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
  if not (x.is_contiguous() and w.is_contiguous() and out.is_contiguous()):
    raise KernelError("linear_tc: operands must be contiguous")
  if M == 0:
    return
  lib = common_lib()
  status = workspace.zeros("gemm_tc_status", 1, torch.int32)
  _check(lib, lib.mi_gemm_tc_bf16(_ptr(out), _ptr(x), _ptr(w), M, N, K, N, _ptr(status, torch.int32), _tc_pairs(), _stream()))


def glu_mul(out: torch.Tensor, gate_up: torch.Tensor, glu: str = "silu", limit: float = 0.0) -> None:
  """out[t, i] = act(gate_up[t, i]) * gate_up[t, I + i] with the gated activation ``glu`` (see ``routed_experts``)."""
  lib = common_lib()
  T, I = out.shape
  if gate_up.shape != (T, 2 * I) or gate_up.dtype != out.dtype:
    raise KernelError("glu_mul: shapes or dtypes do not match")
  kind, lim = _glu(glu, limit)
  _check(lib, lib.mi_glu_mul(_ptr(out), _ptr(gate_up), _dt(out), T, I, kind, lim, _stream()))


def linear_glu(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, workspace, glu: str = "silu", limit: float = 0.0) -> None:
  """out[M, I] = act(x @ w[:I]^T) * (x @ w[I:]^T): the gate-and-up product of a gated feed-forward with the activation
  ``glu``.  ``silu`` is ``linear_swiglu``; the others take the few-row mma.sync kernel with the activation in its epilogue up to 16
  rows, the tcgen05 kernel with the activation in its epilogue from the same number of rows on as SwiGLU, and the product
  followed by the activation kernel between."""
  if glu == "silu":
    linear_swiglu(out, x, w, workspace)
    return
  M, K = x.shape
  I = out.shape[1]
  if w.shape != (2 * I, K) or out.shape[0] != M or out.dtype != x.dtype:
    raise KernelError(f"linear_glu: shapes do not match: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
  if M == 0:
    return
  kind, lim = _glu(glu, limit)
  if (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and M <= SKINNY_BEST_M and K % 8 == 0 and x.is_contiguous() and w.is_contiguous()
      and out.is_contiguous()):
    lib = common_lib()      # few rows: the weight-streaming product with the activation in its epilogue
    _check(lib, lib.mi_gemm_skinny_glu_bf16(_ptr(out), _ptr(x), _ptr(w), M, I, K, I, kind, lim, _stream()))
    return
  many = M >= (GEMM_TC_MIN_M if K >= 4096 else GEMM_TC_MIN_M_NARROW)
  if (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and many and K >= 64 and K % 8 == 0 and I % 8 == 0
      and x.is_contiguous() and w.is_contiguous() and out.is_contiguous() and os.environ.get("MINIINFER_B200_GEMM_TC", "1") != "0"):
    lib = common_lib()
    status = workspace.zeros("gemm_tc_status", 1, torch.int32)
    _check(lib, lib.mi_gemm_tc_glu_bf16(_ptr(out), _ptr(x), _ptr(w), M, I, K, I, _ptr(status, torch.int32), _tc_pairs(), kind, lim, _stream()))
    return
  gu = workspace.buffer("gate_up", (M, 2 * I), x.dtype)
  linear(gu, x, w)
  glu_mul(out, gu, glu, limit)


def silu_mul(out: torch.Tensor, gate_up: torch.Tensor) -> None:
  lib = common_lib()
  T, I = out.shape
  if gate_up.shape != (T, 2 * I) or gate_up.dtype != out.dtype:
    raise KernelError("silu_mul: shapes or dtypes do not match")
  _check(lib, lib.mi_silu_mul(_ptr(out), _ptr(gate_up), _dt(out), T, I, _stream()))


def sample(out: torch.Tensor, logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, seed: torch.Tensor, counter: torch.Tensor, workspace=None) -> None:
  """One token per row of float32 logits; see ``sampling/sampler.py`` for the rule.  ``workspace``
  (a ``Workspace``) lends the scratch for the per-slice results; without it scratch is allocated."""
  lib = common_lib()
  R, V = logits.shape
  for t in (out, temperature, top_k, top_p, seed, counter):
    if t.shape[0] != R:
      raise KernelError("sample: per-row arguments differ in length")
  if R == 0:
    return
  slices = max(1, min(64, 640 // R, -(-V // 1024)))   # about four blocks of the pick kernel per SM
  words = R + 2 * R * slices
  if workspace is not None:
    scratch = workspace.buffer("sample_partials", (words,), torch.int32)
    arrivals = workspace.zeros("sample_arrivals", R, torch.int32)
  else:
    scratch = torch.empty(words, dtype=torch.int32, device=logits.device)
    arrivals = torch.zeros(R, dtype=torch.int32, device=logits.device)
  _check(lib, lib.mi_sample(_ptr(out, torch.int32), _ptr(logits, torch.float32), _ptr(temperature, torch.float32),
                            _ptr(top_k, torch.int32), _ptr(top_p, torch.float32), _ptr(seed, torch.int64),
                            _ptr(counter, torch.int64), _ptr(scratch), _ptr(arrivals, torch.int32), R, V, slices,
                            _stream()), kernels=2)


class AttentionBatch:
  """Device-side description of a step for the attention kernels (all int32).

  ``token_item[t]``: the batch item of token t; ``positions[t]``: its position in its request;
  ``seq_slot[b]``: the block-table row of item b; ``q_start[b]``, ``q_len[b]``, ``ctx_len[b]``:
  the item's first row, its number of new tokens and its length including them.
  Lists the launchers need: ``prefill_tiles`` ((item, first row) of every ``PREFILL_TILE`` rows of the items
  with several new tokens), ``prefill_wide_tiles`` (the same in steps of ``PREFILL_WIDE_TILE``; optional: without it
  the tcgen05 prefill kernel never pairs blocks), ``decode_items`` (the items with exactly one new token), their
  lengths and the largest context."""

  __slots__ = ("token_item", "positions", "seq_slot", "q_start", "q_len", "ctx_len", "num_tokens", "num_items",
               "prefill_tiles", "num_prefill_tiles", "prefill_wide_tiles", "num_prefill_wide_tiles", "decode_items", "num_decode",
               "max_ctx_len", "decode_chunk", "scratch")

  def __init__(self, **kw):
    for k in self.__slots__:
      setattr(self, k, kw.get(k))


def attention(out: torch.Tensor, qkv: torch.Tensor, kv_layer: torch.Tensor, block_table: torch.Tensor,
              batch: AttentionBatch, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
              window: Optional[int], force_generic: bool = False, sink: Optional[torch.Tensor] = None,
              gate: Optional[torch.Tensor] = None, gate_offset: int = 0, out_hd: Optional[int] = None,
              keep_first: int = 0, softcap: float = 0.0, score_bias: Optional[torch.Tensor] = None) -> None:
  """out[t, h*hd:(h+1)*hd] = softmax(scale * q . K^T over the keys the token may see) V, reading
  K and V through the block table.  ``qkv`` holds the step's fused rows; q is its first part.

  Options: ``sink [heads]`` float32 - a learned logit per query head whose exponential joins the softmax's denominator
  once, unscaled, with no key and no value; ``gate`` - rows ``[tokens, width]`` whose columns from ``gate_offset`` on hold,
  head after head, a gate for every output value: the output is multiplied with its sigmoid; ``out_hd`` - only the first
  ``out_hd`` values of each head are written, ``out`` being ``[tokens, heads * out_hd]`` (cache rows padded to ``head_dim``);
  ``keep_first`` - with a window, every token also sees the first ``keep_first`` keys of its request; ``softcap`` > 0 - a
  scaled score ``s`` becomes ``softcap * tanh(s / softcap)``; ``score_bias [heads]`` float32 - no softmax: the weight of a
  visible key is ``sigmoid(s + score_bias[head])``, not normalised over the keys (no sink then)."""
  T = qkv.shape[0]
  ohd = head_dim if out_hd is None else int(out_hd)
  if out.shape != (T, num_heads * ohd) or out.dtype != qkv.dtype or kv_layer.dtype != qkv.dtype or not (0 < ohd <= head_dim):
    raise KernelError("attention: shapes or dtypes do not match")
  page_size = kv_layer.shape[3]
  if kv_layer.shape[1:] != (2, num_kv_heads, page_size, head_dim):
    raise KernelError(f"attention: cache layer has shape {tuple(kv_layer.shape)}")
  if sink is not None and (sink.shape != (num_heads,) or sink.dtype != torch.float32):
    raise KernelError("attention: the sinks must be one float32 per query head")
  gate_stride = 0
  if gate is not None:
    gate_stride = gate.shape[1]
    if gate.dtype != qkv.dtype or gate.shape[0] != T or gate_offset + num_heads * ohd > gate_stride or not gate.is_contiguous():
      raise KernelError("attention: the gate rows do not match")
  if score_bias is not None and (score_bias.shape != (num_heads,) or score_bias.dtype != torch.float32 or sink is not None):
    raise KernelError("attention: the score biases must be one float32 per query head, and go without sinks")
  if softcap < 0:
    raise KernelError(f"attention: softcap={softcap} must not be negative")
  opts = _AttentionOptions(sink, gate, gate_offset, gate_stride, ohd)
  opts.softcap, opts.score_bias = float(softcap), score_bias
  win = int(window) if window else 0
  opts.keep_first = int(keep_first) if win else 0
  even = ohd % 2 == 0 and gate_offset % 2 == 0 and gate_stride % 2 == 0
  if qkv.dtype == torch.bfloat16 and not force_generic and head_dim % 16 == 0 and 16 <= head_dim <= 256 and even:
    _attention_bf16(out, qkv, kv_layer, block_table, batch, num_heads, num_kv_heads, head_dim, scale, win, page_size, opts)
    return
  lib = common_lib()
  _check(lib, lib.mi_attention_generic(
    _ptr(out), _ptr(qkv), qkv.shape[1], _dt(qkv), _ptr(kv_layer), _ptr(block_table, torch.int32),
    block_table.shape[1], _ptr(batch.token_item, torch.int32), _ptr(batch.positions, torch.int32),
    _ptr(batch.seq_slot, torch.int32), T, num_heads, num_kv_heads, head_dim, page_size,
    ctypes.c_float(scale), win, opts.sink_ptr(), opts.gate_ptr(), gate_stride, ohd, opts.keep_first, ctypes.c_float(opts.softcap),
    opts.score_bias_ptr(), _stream()))


class _AttentionOptions:
  """The optional sink, output gate and output width of an attention call, as the kernels take them."""

  __slots__ = ("sink", "gate", "gate_offset", "gate_stride", "out_hd", "keep_first", "softcap", "score_bias")

  def __init__(self, sink, gate, gate_offset, gate_stride, out_hd, keep_first=0):
    self.sink, self.gate, self.gate_offset, self.gate_stride, self.out_hd = sink, gate, gate_offset, gate_stride, out_hd
    self.keep_first = keep_first
    self.softcap, self.score_bias = 0.0, None

  def shaped_scores(self) -> bool:
    return self.softcap > 0 or self.score_bias is not None

  def score_bias_ptr(self):
    return _ptr(self.score_bias, torch.float32) if self.score_bias is not None else _ptr(None)

  def plain(self, head_dim: int) -> bool:
    return self.sink is None and self.gate is None and self.out_hd == head_dim

  def sink_ptr(self):
    return _ptr(self.sink, torch.float32) if self.sink is not None else _ptr(None)

  def gate_ptr(self):
    if self.gate is None:
      return _ptr(None)
    return ctypes.c_void_p(self.gate.data_ptr() + self.gate_offset * self.gate.element_size())


def _rope_in_attention(qkv, cos_sin, kv_layer, batch, nh, nkv, hd, win, page_size) -> int:
  """The cluster size with which a step takes the decode kernel that norms, rotates and stores itself, or 0: a step
  of decode tokens only, bfloat16, head size 128 with the whole head rotated, and few enough (request, kv head)
  pairs for the cluster-scheduled kernel."""
  if not (qkv.is_cuda and qkv.dtype == torch.bfloat16 and hd == 128 and page_size % 64 == 0 and nh // nkv <= 8):
    return 0
  if batch.num_prefill_tiles or batch.num_decode != qkv.shape[0] or batch.num_decode == 0:
    return 0
  if cos_sin is not None and (cos_sin.shape[1] != hd or cos_sin.dtype != torch.float32 or not cos_sin.is_contiguous()):
    return 0
  if os.environ.get("MINIINFER_B200_ROPE_IN_ATTENTION", "1") == "0" or os.environ.get("MINIINFER_B200_DECODE_TMA", "1") == "0":
    return 0
  lib = attention_lib(hd)
  span = min(batch.max_ctx_len, win) if win else batch.max_ctx_len
  return decode_cluster_size(lib, hd, batch.num_decode, nkv, span)


def rope_store_attention(out: torch.Tensor, qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                         cos_sin: Optional[torch.Tensor], positions: torch.Tensor, slot_mapping: Optional[torch.Tensor],
                         kv_layer: torch.Tensor, writes: bool, block_table: torch.Tensor, batch: AttentionBatch,
                         num_heads: int, num_kv_heads: int, head_dim: int, eps: float, scale: float, window: Optional[int]) -> None:
  """From the fused QKV rows of a step to its attention output: ``qk_norm_rope_store`` (which also puts the new
  keys and values into the layer's pages, if ``writes``) followed by ``attention``.  A step of a few decode tokens
  takes one kernel for both (attention_decode_cluster.cu), which does the first step's arithmetic operation for
  operation: the results are the same bit for bit, except that ``qkv`` is then left as the product wrote it."""
  win = int(window) if window else 0
  page_size = kv_layer.shape[3] if kv_layer is not None and kv_layer.dim() == 5 else 0
  cluster = _rope_in_attention(qkv, cos_sin, kv_layer, batch, num_heads, num_kv_heads, head_dim, win, page_size) if page_size else 0
  if not cluster:
    qk_norm_rope_store(qkv, q_weight, k_weight, cos_sin, positions, slot_mapping if writes else None,
                       kv_layer if writes else None, num_heads, num_kv_heads, head_dim, eps)
    attention(out, qkv, kv_layer, block_table, batch, num_heads, num_kv_heads, head_dim, scale, window)
    return
  T = qkv.shape[0]
  if out.shape != (T, num_heads * head_dim) or out.dtype != qkv.dtype or kv_layer.dtype != qkv.dtype:
    raise KernelError("rope_store_attention: shapes or dtypes do not match")
  if kv_layer.shape[1:] != (2, num_kv_heads, page_size, head_dim) or qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
    raise KernelError(f"rope_store_attention: cache layer {tuple(kv_layer.shape)} or qkv {tuple(qkv.shape)} do not match the head counts")
  lib = attention_lib(head_dim)
  if batch.scratch is not None:
    status = batch.scratch.zeros("attention_decode_counters", batch.num_decode * num_kv_heads + 1, torch.int32)[:1]
  else:
    status = torch.zeros(1, dtype=torch.int32, device=qkv.device)
  none = _ptr(None)
  _check(lib, lib.mi_attention_decode_cluster_rope(
    _ptr(out), _ptr(qkv), qkv.shape[1], _kv_tensor_map(lib, kv_layer), _ptr(block_table, torch.int32), block_table.shape[1],
    none, _ptr(batch.q_start, torch.int32), _ptr(batch.ctx_len, torch.int32),     # no list of decode items: all items are, in order (one dependent load less before the first copy: 0.4 % of a step)
    _ptr(batch.seq_slot, torch.int32), _ptr(status, torch.int32), batch.num_decode, num_heads, num_kv_heads, page_size,
    ctypes.c_float(scale), win, cluster, batch.max_ctx_len,
    _ptr(q_weight, torch.float32) if q_weight is not None else none, _ptr(k_weight, torch.float32) if k_weight is not None else none,
    _ptr(cos_sin, torch.float32) if cos_sin is not None else none,
    _ptr(slot_mapping, torch.int32) if (writes and slot_mapping is not None) else none,
    _ptr(kv_layer) if writes else none, ctypes.c_float(eps), _stream()))
  if batch.scratch is None and int(status[0]) != 0:
    raise KernelError("attention_decode_cluster: a bounded wait on a copy barrier ran out")


DECODE_CHUNKS = (512, 256, 128, 64)
def decode_chunk(num_decode: int, num_kv_heads: int, max_ctx_len: int, head_dim: int) -> int:
  """Keys per block of the cp.async split-KV decode kernel: the longest chunk that still gives every
  SM about two blocks, so that a small batch is spread over the whole GPU."""
  forced = os.environ.get("MINIINFER_B200_DECODE_CHUNK")
  if forced:
    return int(forced)
  two_per_sm = 2 * _num_sms(torch.device("cuda", torch.cuda.current_device()))
  for c in DECODE_CHUNKS:
    if num_decode * num_kv_heads * -(-max_ctx_len // c) >= two_per_sm:
      return c
  return DECODE_CHUNKS[-1]


_cluster_fit: Dict[tuple, int] = {}


def decode_cluster_size(lib, head_dim: int, num_decode: int, num_kv_heads: int, span: int) -> int:
  """Blocks per (request, kv head) for the cluster-scheduled decode kernel (attention_decode_cluster.cu), or 0 if
  the step should take the persistent kernel instead.  The largest cluster (16, 8, 4, 2, 1 blocks) that leaves a
  block at least one 64-key tile (6 is tried as well: two requests are a little faster with it) and whose clusters - one per (request, kv head) - can all be on the GPU at once:
  a second round of clusters would double the kernel's time.  (Measured on B200, 8 kv heads of 128, 2048-token
  contexts: 1 / 2 / 4 / 8 / 16 requests are fastest with clusters of 8 / 4 / 4 / 2 / 1, which is what this rule
  picks; decode steps took 0.74 / 0.79 / 0.83 / 0.99 / 1.34 ms against 0.92 / 0.92 / 0.99 / 1.12 / 1.55 ms with
  the persistent kernel, and the sizes were measured again after the cluster's merge had lost a barrier.)  Blocks with more than 64 tiles each, or more (request, kv head) pairs than fit at once,
  stream better from the persistent kernel, which deals the tiles out evenly over the SMs."""
  tiles = -(-span // 64) + 1

  def fit(c: int) -> int:
    key = (head_dim, c, -(-tiles // c))
    n = _cluster_fit.get(key)
    if n is None:
      n = _cluster_fit[key] = int(lib.mi_attention_decode_cluster_fit(c, -(-tiles // c)))
    return n

  forced = os.environ.get("MINIINFER_B200_DECODE_CLUSTER")
  if forced is not None:
    c = int(forced)
    return c if c and fit(c) > 0 else 0
  pairs = num_decode * num_kv_heads
  for c in (16, 8, 6, 4, 2, 1):
    if c <= tiles and -(-tiles // c) <= DECODE_CLUSTER_MAX_TILES_PER_BLOCK and pairs <= fit(c):
      return c
  return 0


DECODE_CLUSTER_MAX_TILES_PER_BLOCK = 64


def _attention_bf16(out, qkv, kv_layer, block_table, batch, nh, nkv, hd, scale, win, page_size, opts=None) -> None:
  """Tensor-core kernel for the items with several new tokens, split-KV kernel for the decode items;
  the two write disjoint rows of ``out``."""
  lib = attention_lib(hd)
  if opts is None:
    opts = _AttentionOptions(None, None, 0, 0, hd)
  # the TMA and tcgen05 kernels write whole heads; sink and gate they take; kept first keys only the tcgen05 prefill kernel knows
  whole_heads = opts.out_hd == hd and not opts.keep_first
  if batch.num_prefill_tiles:
    # the tcgen05 kernel takes sink and gate; its output rows are whole heads, and it reads the gate 16 bytes at a time
    gate_ok = opts.gate is None or (opts.gate_offset % 8 == 0 and opts.gate_stride % 8 == 0 and opts.gate.data_ptr() % 16 == 0)
    use_tc = (opts.out_hd == hd and gate_ok and page_size % 64 == 0 and lib.mi_attention_prefill_tc_supported() == 1
              and os.environ.get("MINIINFER_B200_PREFILL_TC", "1") != "0")
    if use_tc:
      if batch.scratch is not None:
        status = batch.scratch.zeros("attention_prefill_status", 1, torch.int32)
      else:
        status = torch.zeros(1, dtype=torch.int32, device=qkv.device)
      wide, n_wide = batch.prefill_wide_tiles, int(batch.num_prefill_wide_tiles or 0)
      # two blocks on one work (tcgen05 cta_group::2: half the K / V bytes per SM, twice the stages): measured on B200
      # at 16 heads of 128, 291 against 303 us for 8192 new tokens, 31.4 against 31.2 us for 2048 - so only large steps
      force = os.environ.get("MINIINFER_B200_PREFILL_PAIRS")
      pairs = int(force == "1") if force in ("0", "1") else int(n_wide >= PREFILL_PAIRS_MIN_WIDE_TILES)
      _check(lib, lib.mi_attention_prefill_tc(
        _ptr(out), _qkv_tensor_map(lib, qkv), _kv_tensor_map(lib, kv_layer), _ptr(block_table, torch.int32), block_table.shape[1],
        _ptr(batch.prefill_tiles, torch.int32), batch.num_prefill_tiles, _ptr(batch.q_start, torch.int32),
        _ptr(batch.q_len, torch.int32), _ptr(batch.ctx_len, torch.int32), _ptr(batch.seq_slot, torch.int32),
        _ptr(status, torch.int32), nh, nkv, page_size, ctypes.c_float(scale), win, _num_sms(qkv.device), _stream(),
        _ptr(wide, torch.int32) if wide is not None else _ptr(None), n_wide, pairs,
        opts.sink_ptr(), opts.gate_ptr(), opts.gate_stride, opts.keep_first, ctypes.c_float(opts.softcap), opts.score_bias_ptr()))
      if batch.scratch is None and int(status[0]) != 0:
        raise KernelError("attention_prefill_tc: a bounded wait on a barrier ran out")
    else:
      _check(lib, lib.mi_attention_prefill_bf16(
        _ptr(out), _ptr(qkv), qkv.shape[1], _ptr(kv_layer), _ptr(block_table, torch.int32), block_table.shape[1],
        _ptr(batch.prefill_tiles, torch.int32), batch.num_prefill_tiles, _ptr(batch.q_start, torch.int32),
        _ptr(batch.q_len, torch.int32), _ptr(batch.ctx_len, torch.int32), _ptr(batch.seq_slot, torch.int32),
        nh, nkv, page_size, ctypes.c_float(scale), win, opts.sink_ptr(), opts.gate_ptr(), opts.gate_stride, opts.out_hd,
        opts.keep_first, ctypes.c_float(opts.softcap), opts.score_bias_ptr(), _stream()))
  if batch.num_decode:
    span = min(batch.max_ctx_len, win) if win else batch.max_ctx_len
    G = nh // nkv
    tma_shapes = whole_heads and hd % 64 == 0 and page_size % 64 == 0 and os.environ.get("MINIINFER_B200_DECODE_TMA", "1") != "0"
    # shaped scores (a cap, sigmoid weights) the persistent TMA kernel and the cp.async kernel know, the cluster kernel does not
    cluster = decode_cluster_size(lib, hd, batch.num_decode, nkv, span) if (tma_shapes and G <= 8 and not opts.shaped_scores()) else 0
    if cluster:
      if batch.scratch is not None:
        status = batch.scratch.zeros("attention_decode_counters", batch.num_decode * nkv + 1, torch.int32)[:1]
      else:
        status = torch.zeros(1, dtype=torch.int32, device=qkv.device)
      _check(lib, lib.mi_attention_decode_cluster(
        _ptr(out), _ptr(qkv), qkv.shape[1], _kv_tensor_map(lib, kv_layer), _ptr(block_table, torch.int32), block_table.shape[1],
        _ptr(batch.decode_items, torch.int32), _ptr(batch.q_start, torch.int32), _ptr(batch.ctx_len, torch.int32),
        _ptr(batch.seq_slot, torch.int32), _ptr(status, torch.int32), batch.num_decode, nh, nkv, page_size, ctypes.c_float(scale), win,
        cluster, batch.max_ctx_len, _stream(), opts.sink_ptr(), opts.gate_ptr(), opts.gate_stride))
      if batch.scratch is None and int(status[0]) != 0:
        raise KernelError("attention_decode_cluster: a bounded wait on a copy barrier ran out")
      return
    # more than 8 query heads per kv head: the TMA kernel would walk an item's tiles twice and hand a stage back only
    # in the second pass, which cannot work once an item has more tiles than there are stages - the cp.async kernel takes those
    use_tma = (whole_heads and hd % 64 == 0 and page_size % 64 == 0 and G <= 8 and os.environ.get("MINIINFER_B200_DECODE_TMA", "1") != "0")
    if use_tma:
      # the TMA kernel deals 64-key tiles out evenly; a (request, kv head) is cut into at most as many
      # pieces as it has tiles, and no more than there are blocks
      chunk = 64
      max_splits = min(-(-span // 64) + 2, _num_sms(qkv.device))
    else:
      chunk = batch.decode_chunk or decode_chunk(batch.num_decode, nkv, span, hd)
      max_splits = -(-span // chunk) + 1 + -(-opts.keep_first // chunk)
    n = batch.num_decode * nh * max_splits * (hd + 2)
    if batch.scratch is not None:
      scratch = batch.scratch.buffer("attention_decode_partials", (n,), torch.float32)
      counters = batch.scratch.zeros("attention_decode_counters", batch.num_decode * nkv + 1, torch.int32)
    else:
      scratch = torch.empty(n, dtype=torch.float32, device=qkv.device)
      counters = torch.zeros(batch.num_decode * nkv + 1, dtype=torch.int32, device=qkv.device)
    if use_tma:
      _check(lib, lib.mi_attention_decode_tma(
        _ptr(out), _ptr(qkv), qkv.shape[1], _kv_tensor_map(lib, kv_layer), _ptr(block_table, torch.int32), block_table.shape[1],
        _ptr(batch.decode_items, torch.int32), _ptr(batch.q_start, torch.int32), _ptr(batch.ctx_len, torch.int32),
        _ptr(batch.seq_slot, torch.int32), _ptr(scratch, torch.float32), _ptr(counters[1:], torch.int32), _ptr(counters[:1], torch.int32),
        batch.num_decode, nh, nkv, page_size, ctypes.c_float(scale), win, chunk, max_splits, _num_sms(qkv.device), _stream(),
        opts.sink_ptr(), opts.gate_ptr(), opts.gate_stride, ctypes.c_float(opts.softcap), opts.score_bias_ptr()))
      if batch.scratch is None and int(counters[0]) != 0:
        raise KernelError("attention_decode_tma: a bounded wait on a copy barrier ran out")
    else:
      _check(lib, lib.mi_attention_decode_bf16(
        _ptr(out), _ptr(qkv), qkv.shape[1], _ptr(kv_layer), _ptr(block_table, torch.int32), block_table.shape[1],
        _ptr(batch.decode_items, torch.int32), _ptr(batch.q_start, torch.int32), _ptr(batch.ctx_len, torch.int32),
        _ptr(batch.seq_slot, torch.int32), _ptr(scratch, torch.float32), _ptr(counters[1:], torch.int32),
        batch.num_decode, nh, nkv, page_size, ctypes.c_float(scale), win, chunk, max_splits,
        opts.sink_ptr(), opts.gate_ptr(), opts.gate_stride, opts.out_hd, opts.keep_first, ctypes.c_float(opts.softcap),
        opts.score_bias_ptr(), _stream()))


_tensor_maps: Dict[tuple, ctypes.Array] = {}
_sm_counts: Dict[int, int] = {}


def _num_sms(device) -> int:
  idx = device.index if device.index is not None else torch.cuda.current_device()
  if idx not in _sm_counts:
    _sm_counts[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
  return _sm_counts[idx]


def _kv_tensor_map(lib, kv_layer: torch.Tensor):
  """The TMA descriptor of a cache layer (made once per layer: it holds the layer's address)."""
  key = (kv_layer.data_ptr(), tuple(kv_layer.shape))
  m = _tensor_maps.get(key)
  if m is None:
    m = ctypes.create_string_buffer(128)
    rows = kv_layer.shape[0] * kv_layer.shape[1] * kv_layer.shape[2] * kv_layer.shape[3]
    code = lib.mi_kv_tensor_map(m, _ptr(kv_layer), ctypes.c_longlong(rows))
    if code != 0:
      raise KernelError(lib.mi_last_error().decode())
    _tensor_maps[key] = m
  return m


def _qkv_tensor_map(lib, qkv: torch.Tensor):
  """The TMA descriptor of a step's fused QKV rows (kept per address and shape: the workspace hands
  out the same buffer step after step)."""
  key = ("qkv", qkv.data_ptr(), tuple(qkv.shape))
  m = _tensor_maps.get(key)
  if m is None:
    if not qkv.is_contiguous():
      raise KernelError("attention: the QKV rows must be contiguous")
    if len(_tensor_maps) > 4096:
      _tensor_maps.clear()
    m = ctypes.create_string_buffer(128)
    code = lib.mi_qkv_tensor_map(m, _ptr(qkv), ctypes.c_longlong(qkv.shape[0]), ctypes.c_longlong(qkv.shape[1]))
    if code != 0:
      raise KernelError(lib.mi_last_error().decode())
    _tensor_maps[key] = m
  return m


def forget_tensors() -> None:
  """Drops what this module keeps per tensor address (transposed views of weights, TMA descriptors of cache
  layers and QKV buffers).  The views keep the weights' memory alive: an engine that is done calls this so
  that its memory can go back to the device."""
  _transposed_views.clear()
  _tensor_maps.clear()


def device_status(ws) -> int:
  """The status words that kernels with bounded waits set when a wait ran out (0: all well)."""
  code = 0
  for name in ("attention_decode_counters", "attention_prefill_status", "gemm_tc_status"):
    buf = ws._bufs.get((name, torch.int32))
    if buf is not None:
      code |= int(buf[0])
  for _, _, status in _stream_ws.values():
    code |= int(status[0])
  return code
