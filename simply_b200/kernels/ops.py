"""The kernel table: every device operation the engine's parts call.

`CudaOps(dtype)` is the only implementation in the package.  It needs a CUDA
device and the compiled library and raises if either is missing; there is no
CPU path.  `dtype` is the activation and cache dtype: `torch.bfloat16` is the
serving path, `torch.float32` runs the whole model in true 32-bit arithmetic on
CUDA cores (own SIMT matrix product, no tensor-core mode).

Matrix products: in bfloat16, steps with at most 16 tokens use the engine's own
weight-streaming kernel (with fused soft-cap or gated-activation epilogues);
larger ones go to the library product (cuBLAS through torch.mm), as the
reference leaves them to XLA.  Everything else (attention over the paged cache,
norms, rotation, cache write, activation, embedding, sampling) is hand-written.
"""

from __future__ import annotations

import ctypes
import os
from typing import Any, Sequence

import numpy as np
import torch

from simply_b200.kernels import build

_F32, _BF16 = 0, 1
_ERRORS = {
    1: "a block-table entry outside the page pool was about to be followed",
    2: "a token id outside the embedding table",
    4: "a gather row outside the batch",
    8: "a wait for a bulk copy timed out",
    16: "a state slot outside the state tensor",
}
_STATUS = {
    -2: "row too wide for the norm kernel's shared-memory buffer",
    -3: "unsupported cast",
    -4: "head size must be even",
    -5: "unknown activation code",
    -6: "too many rows for one launch of the float32 product",
    -7: "head size outside the attention kernel's range",
    -8: "query heads are no multiple of key/value heads",
    -9: "shape outside the weight-streaming product's range",
    -10: "batch outside the decode-advance kernel's range",
    -11: "head size does not allow a tensor map",
    -12: "the driver refused to encode a tensor map",
    -13: "sizes outside the recurrent-mixer kernels' range",
}


def _code(t: torch.Tensor) -> int:
  if t.dtype == torch.float32:
    return _F32
  if t.dtype == torch.bfloat16:
    return _BF16
  raise TypeError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _ptr(t: torch.Tensor | None):
  """The tensor's address as the plain integer that a declared `c_void_p` parameter takes (every
  entry point's parameter types are declared; None is the null pointer)."""
  return None if t is None else t.data_ptr()


class KernelError(RuntimeError):
  pass


class _HeldStream:

  def __init__(self, ops):
    self.ops = ops

  def __enter__(self):
    self.previous = self.ops._step_stream
    self.ops._step_stream = ctypes.c_void_p(torch.cuda.current_stream(self.ops.device).cuda_stream)

  def __exit__(self, *exc):
    self.ops._step_stream = self.previous


class AttentionGraphPlan:
  """Static work list of the split-key attention kernel for decode bursts replayed from a CUDA
  graph, for one kind of attention layer (see `Mixer.graph_plans` for the interface).

  Every sequence gets the same number of work items, so the launch has a fixed size: the chunks
  that hold keys between the lowest key visible at the burst's first step and the highest at its
  last, then fillers.  The words are: items [batch * per_seq, 2], split_start [batch],
  split_count [batch]."""

  def __init__(self, ops: "CudaOps", window: int | None, group: int, num_kv_heads: int, head_dim: int,
               batch: int, bucket: int, max_burst: int, page_size: int):
    self.key = ops._plan_key(window, group, num_kv_heads, head_dim, page_size)
    self.window, self.group, self.batch = window, group, batch
    # Most keys a sequence of this bucket sees in such a layer during a burst.
    span = min(bucket, window + max_burst + 64) if window else bucket
    self.chunk = ops.decode_chunk_for([bucket - span] * batch, [bucket] * batch, num_kv_heads, head_dim)
    self.per_seq = -(-span // self.chunk) + 1
    self.words = batch * self.per_seq * 2 + 2 * batch

  def bind(self, view: torch.Tensor) -> dict:
    n = self.batch * self.per_seq * 2
    return dict(num_prefill=0, num_decode=self.batch * self.per_seq, chunk=self.chunk, rows_max=self.group,
                rows_per_tile=64, prefill_items=None, decode_items=view[:n],
                split_start=view[n:n + self.batch], split_count=view[n + self.batch:])

  def fill(self, host_words: np.ndarray, lengths: np.ndarray, steps: int) -> None:
    items, start, count = CudaOps.static_decode_plan(lengths, steps, self.window, self.chunk, self.per_seq)
    n = items.size
    host_words[:n] = items.reshape(-1)
    host_words[n:n + self.batch] = start
    host_words[n + self.batch:] = count

  def ranges(self, lengths: np.ndarray, steps: int):
    return CudaOps.decode_chunk_range(lengths, steps, self.window, self.chunk)


class PooledAttentionGraphPlan:
  """Static work list for attention with pooled blocks in a decode graph: every request brings one
  token and is one tile of the prefill kernel, so the list is (request, 0) for each and never changes."""

  def __init__(self, key: tuple, batch: int):
    self.key, self.batch, self.words = key, batch, 2 * batch

  def bind(self, view: torch.Tensor) -> dict:
    return dict(num_prefill=self.batch, num_decode=0, rows_per_tile=64, prefill_items=view[:2 * self.batch])

  def fill(self, host_words: np.ndarray, lengths: np.ndarray, steps: int) -> None:
    host_words[:2 * self.batch] = np.stack([np.arange(self.batch), np.zeros(self.batch, dtype=np.int64)], axis=1).reshape(-1)

  def ranges(self, lengths: np.ndarray, steps: int):
    return ()


class CudaOps:

  name = "cuda"
  # Largest token count the weight-streaming product for a handful of tokens takes, and the largest
  # the one for a serving batch takes (csrc/gemm_skinny_bf16.cu, csrc/gemm_stream_tc.cu).
  skinny_max_rows = 16
  mid_max_rows = 128

  def __init__(self, dtype: torch.dtype = torch.bfloat16, device: str | torch.device = "cuda"):
    if dtype not in (torch.float32, torch.bfloat16):
      raise TypeError(f"activation dtype must be float32 or bfloat16, got {dtype}")
    if not torch.cuda.is_available():
      raise KernelError("simply_b200 needs a CUDA device (sm_100a); there is no CPU path")
    self.dtype = dtype
    self.device = torch.device(device)
    self.lib = build.load()
    major, minor = torch.cuda.get_device_capability(self.device)
    if major != 10:
      raise KernelError(f"kernels are built for sm_100a; this device is sm_{major}{minor}")
    self._declare()
    self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
    self._attn_fns: dict[int, tuple] = {}
    self._latent_fns: dict[tuple[int, int], Any] = {}
    self._tensor_maps: dict[tuple, tuple] = {}
    # Work counter of the split-key attention kernel: zero between launches (its merge kernel resets it).
    self._attn_counter = torch.zeros(1, dtype=torch.int32, device=self.device)
    # bfloat16 attention runs on tensor cores where the shape allows; False forces the general kernel.
    self.tensor_core_attention = True
    # Split-key attention: the chunk length is chosen so that the work items fill the kernel's
    # persistent grid evenly; decode_chunk > 0 fixes it instead (a multiple of 64).
    self.decode_chunk = 0
    self._decode_slots: dict[int, int] = {}
    # 0: the kernel is picked by the number of query rows; 1 forbids TMA; 16 forces the 16-row kernel (tests).
    self.decode_variant = 0
    self.direct_library_products = True  # False: through torch.mm
    self._library_workspaces: dict = {}
    self._step_stream = None
    # 0: prefill tiles of 64 query rows; 64 or 128 forces a size.
    self.prefill_rows = 0
    # Prefill attention on the tcgen05 tensor cores where the shapes allow (head size a multiple of
    # 64, group dividing 128, page size a power of two); False keeps the mma.sync kernel.
    self.prefill_tcgen05 = True
    # ... and there by pairs of blocks (cta_group::2) where the shapes allow (head size 128 or 256,
    # pages of at least 64 tokens); False keeps single blocks (tests).
    self.prefill_pairs = True
    self._rounded_scales: dict[float, float] = {}
    # Routed experts: from this many rows per expert on average (and outside graph capture) a
    # step's experts run one by one through the products of a dense feed-forward, after one look
    # at how many rows each got; below, and in decode graphs, the grouped kernel (csrc/moe.cu)
    # serves them without the host.  0: always the grouped kernel.
    self.expert_rows_for_dense_products = int(os.environ.get("SIMPLY_B200_EXPERT_DENSE_ROWS", "384"))
    self.expert_side_stream = True  # False: all experts on the step's stream (tests, experiments)
    self._wide_tables: dict[tuple, torch.Tensor] = {}
    self.prefill_single_key_group = False  # True: 64-row tiles with 4 warps instead of 4 x 2 (experiments, tests)
    # 0: the weight-streaming product picks its warps per block; 4, 8 or 16 forces them (experiments).
    self.skinny_warps = 0
    # False keeps the q, k, v projection and the rotation + cache write as two kernels (tests).
    self.fused_qkv_rope = True
    # False sends steps of 17 to 64 tokens to the library product (tests, experiments); mid_split
    # fixes the number of blocks that share a row tile's k (0: the launch chooses).
    self.mid_rows_kernel = True
    # Most rows for which each kind of product takes that kernel rather than the library's: the
    # fused q, k, v projection, the gated product, a plain product, the output layer.  The kernel
    # takes up to 128 rows; measured inside decode steps of the Gemma 2 2B shape it is ahead of
    # the library's products up to 32 rows (by 1 to 2 % of the step) and behind them from 33
    # (by 1 to 4 %), so that is where the line is drawn.
    # From this many tokens the gated feed-forward product runs on the engine's own tcgen05 kernel
    # with the activation on the accumulators (csrc/gemm_gated_tc.cu); below, and for shapes it
    # does not take, the library's product and a pass of its own for the activation.  0: never.
    self.gated_tc_min_rows = int(os.environ.get("SIMPLY_B200_GATED_TC_MIN_ROWS", "129"))
    self.gated_tc_blocks = 0  # 0: one block per SM (tests: fewer, so that blocks walk many tiles)
    # Blocks work in pairs (tcgen05 cta_group::2, tiles of 256 tokens); False: each alone on tiles
    # of 128 (tests).  Measured at the Gemma 2 shapes: in short bursts single blocks are ahead on
    # the largest products (by 3 to 5 %), but whenever the GPU runs long enough for the power limit
    # to set the clocks (a prefill step of the 27B shape is 90 ms) pairs, which move a third less
    # data, are ahead at every size (by 2 to 4 %).
    self.gated_tc_pairs = True
    self.mid_rows = {"qkv": 32, "gated": 32, "plain": 32, "head": 32}
    env = os.environ.get("SIMPLY_B200_SERVING_BATCH_PRODUCT")  # experiments: "qkv:128,gated:32,plain:0,head:128"
    if env:
      for item in env.split(","):
        name, _, rows = item.partition(":")
        self.mid_rows[name] = int(rows or 128)
    self.mid_split = 0
    self.mid_stages = 0  # 0: the launch chooses the depth of the ring of stages; 8 deep, 4 shallow (tests)
    # The true 32-bit path must not be routed through a reduced-precision matrix mode.
    torch.backends.cuda.matmul.allow_tf32 = False
    self.launches = 0

  # ---- plumbing -------------------------------------------------------------
  def _declare(self) -> None:
    c_int, c_float, c_void, c_ll = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong
    protos = {
        "sb_embed": [c_void, c_int, c_void, c_float, c_void, c_int, c_int, c_int, c_void, c_void],
        "sb_residual_norm": [c_void, c_void, c_void, c_int, c_void, c_int, c_float, c_int, c_void, c_int, c_float,
                             c_int, c_void, c_void, c_int, c_int, c_int, c_void, c_void],
        "sb_rms_norm": [c_void, c_int, c_void, c_int, c_float, c_int, c_void, c_int, c_int, c_int, c_void],
        "sb_gather_rows": [c_void, c_int, c_void, c_void, c_int, c_int, c_int, c_void, c_void],
        "sb_add_to_residual": [c_void, c_void, c_int, c_ll, c_void],
        "sb_cast": [c_void, c_int, c_void, c_int, c_ll, c_void],
        "sb_rotation_tables": [c_void, c_void, c_float, c_void, c_void, c_int, c_int, c_void],
        "sb_rope_cache_write": [c_void, c_int, c_void, c_void, c_float, c_void, c_void, c_void, c_int, c_void,
                                c_void, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void, c_void],
        "sb_gated_activation": [c_void, c_int, c_void, c_int, c_int, c_int, c_float, c_void],
        "sb_soft_cap": [c_void, c_float, c_ll, c_void],
        "sb_gemm_f32_nt": [c_void, c_void, c_void, c_int, c_int, c_int, c_float, c_void],
        "sb_gemm_skinny_bf16": [c_void, c_void, c_void, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void],
        "sb_gemm_skinny_bf16_xielu": [c_void, c_void, c_void, c_int, c_int, c_int, c_float, c_float, c_int, c_void],
        "sb_gemm_stream_tc": [c_void, c_void, c_void, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int,
                              c_void, c_void],
        "sb_gemm_gated_tc": [c_void, c_void, c_void, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void, c_void],
        "sb_qkv_rope_stream_tc": [c_void, c_void, c_int, c_int, c_void, c_void, c_float, c_void, c_void, c_void, c_int,
                                  c_void, c_void, c_int, c_int, c_int, c_int, c_int, c_void, c_int, c_int, c_void],
        "sb_qkv_rope_skinny": [c_void, c_void, c_int, c_int, c_void, c_void, c_float, c_void, c_void, c_void, c_int,
                               c_void, c_void, c_int, c_int, c_int, c_int, c_int, c_void, c_int, c_void],
        "sb_paged_attention_generic": [c_void, c_int, c_void, c_void, c_int, c_void, c_void, c_void, c_int,
                                       c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void, c_void],
        "sb_paged_attention_general": [c_void, c_int, c_void, c_void, c_int, c_void, c_void, c_void, c_int,
                                       c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void, c_void,
                                       c_int, c_int, c_int, c_int, c_void, c_void, c_void, c_void],
        "sb_qk_norm_rotate_store": [c_void, c_int, c_int, c_void, c_void, c_float, c_void, c_void, c_int, c_void,
                                    c_void, c_void, c_void, c_int, c_void, c_void, c_int, c_int, c_int, c_int, c_int,
                                    c_int, c_int, c_int, c_void, c_void],
        "sb_pool_blocks": [c_void, c_int, c_void, c_int, c_int, c_void, c_void, c_int, c_int, c_void, c_void, c_int,
                           c_int, c_int, c_int, c_int, c_int, c_int, c_void, c_void],
        "sb_rotate_heads": [c_void, c_int, c_void, c_void, c_float, c_int, c_int, c_int, c_void, c_void],
        "sb_delta_inputs": [c_void, c_int, c_void, c_int, c_int, c_void, c_void, c_void, c_void, c_void, c_void,
                            c_void, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void, c_void, c_void,
                            c_void, c_void, c_void, c_void],
        "sb_delta_scan": [c_void, c_void, c_void, c_void, c_void, c_void, c_void, c_void, c_int, c_int, c_int,
                          c_int, c_int, c_int, c_int, c_void, c_void, c_void],
        "sb_gated_head_norm": [c_void, c_void, c_int, c_int, c_int, c_void, c_float, c_int, c_int, c_int, c_void,
                               c_void],
        "sb_normed_mean": [c_void, c_void, c_void, c_void, c_void, c_void, c_void, c_void, c_int, c_int, c_float,
                           c_int, c_int, c_void, c_void],
        "sb_rotate_headnorm_store": [c_void, c_int, c_int, c_void, c_float, c_float, c_void, c_int, c_int, c_int, c_int,
                                     c_void, c_void, c_void, c_int, c_void, c_void, c_int, c_int, c_int, c_int,
                                     c_int, c_int, c_int, c_int, c_void, c_void],
        "sb_sigmoid_gate": [c_void, c_void, c_int, c_int, c_int, c_int, c_int, c_void],
        "sb_embed_positions": [c_void, c_void, c_int, c_void, c_void, c_float, c_void, c_int, c_int, c_int, c_int,
                               c_void, c_void],
        "sb_spread_streams": [c_void, c_void, c_int, c_int, c_int, c_void],
        "sb_streams_step": [c_void, c_void, c_int, c_void, c_void, c_void, c_void, c_int, c_float, c_int, c_void,
                            c_int, c_void, c_void, c_int, c_int, c_int, c_void, c_void],
        "sb_short_conv": [c_void, c_int, c_int, c_int, c_void, c_void, c_void, c_void, c_void, c_void, c_int, c_int,
                          c_int, c_int, c_int, c_int, c_int, c_int, c_void, c_void, c_void],
        "sb_group_norm_gate": [c_void, c_void, c_int, c_int, c_int, c_int, c_void, c_float, c_int, c_int, c_int,
                               c_void, c_void],
        "sb_tanh_columns": [c_void, c_int, c_int, c_int, c_int, c_void, c_int, c_void],
        "sb_table_route": [c_void, c_void, c_int, c_int, c_int, c_void, c_void, c_int, c_void, c_void],
        "sb_head_linear": [c_void, c_int, c_int, c_int, c_void, c_int, c_int, c_int, c_int, c_void, c_int, c_int,
                           c_float, c_int, c_void],
        "sb_latent_prepare": [c_void, c_int, c_int, c_void, c_void, c_float, c_void, c_int, c_int, c_int, c_int,
                              c_void, c_void, c_void, c_int, c_int, c_int, c_void, c_void, c_int, c_void, c_void],
        "sb_turn_query_part": [c_void, c_int, c_int, c_void, c_int, c_int, c_int, c_void, c_int, c_int, c_float,
                               c_void, c_int, c_int, c_void],
        "sb_general_delta_scan": [c_void, c_int, c_void, c_int, c_int, c_void, c_void, c_void, c_void, c_void, c_int,
                                  c_int, c_int, c_int, c_int, c_int, c_void, c_void, c_void, c_void],
        "sb_state_space_scan": [c_void, c_int, c_void, c_int, c_int, c_int, c_void, c_void, c_void, c_void, c_void,
                                c_void, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void, c_void,
                                c_void, c_void],
        "sb_forget_scan": [c_void, c_int, c_int, c_void, c_void, c_void, c_void, c_void, c_int, c_int, c_int, c_int,
                           c_int, c_int, c_int, c_void, c_void, c_void, c_void],
        "sb_moe_route": [c_void, c_int, c_int, c_int, c_void, c_void, c_void, c_void, c_int, c_int, c_float, c_int, c_int,
                         c_void, c_void, c_void, c_void],
        "sb_moe_group": [c_void, c_int, c_int, c_int, c_void, c_void, c_void, c_void, c_void, c_void],
        "sb_moe_product": [c_void, c_void, c_int, c_void, c_int, c_int, c_int, c_int, c_void, c_void, c_void, c_int,
                           c_int, c_float, c_void, c_void],
        "sb_scaled_residual_tanh": [c_void, c_void, c_void, c_void, c_void, c_int, c_void, c_void, c_void, c_void,
                                    c_void, c_int, c_int, c_int, c_void, c_void],
        "sb_pack_pair": [c_void, c_void, c_void, c_int, c_int, c_int, c_void],
        "sb_add_row": [c_void, c_void, c_int, c_int, c_void],
        "sb_xielu": [c_void, c_void, c_void, c_int, c_ll, c_void],
        "sb_scale_values": [c_void, c_float, c_ll, c_void],
        "sb_moe_combine": [c_void, c_void, c_int, c_void, c_void, c_void, c_void, c_void, c_int, c_int, c_int, c_int,
                           c_void, c_void],
        "sb_sample": [c_void, c_void, c_void, c_int, c_int, c_void, c_void],
        "sb_sample_logprobs": [c_void, c_void, c_void, c_void, c_void, c_int, c_int, c_void, c_void],
        "sb_decode_advance": [c_void, c_void, c_void, c_void, c_void, c_void, c_void, c_int, c_void],
        "sb_keep_logits": [c_void, c_void, c_void, c_ll, c_void],
    }
    for name, argtypes in protos.items():
      fn = getattr(self.lib, name)
      fn.argtypes = argtypes
      fn.restype = c_int
    self.lib.sb_gemm_library_bf16.argtypes = [c_void, c_void, c_void, c_int, c_int, c_int, c_int, c_void, c_ll, c_void]
    self.lib.sb_gemm_library_bf16.restype = c_int
    self.lib.sb_gemm_library_bf16_heads.argtypes = [c_void, c_int, c_int, c_void, c_void, c_int, c_int, c_int, c_int, c_int,
                                                    c_int, ctypes.c_float, c_void, c_ll, c_void]
    self.lib.sb_gemm_library_bf16_heads.restype = c_int
    c_ip = ctypes.POINTER(c_int)
    self.lib.sb_experts_dense_bf16.argtypes = [c_void, c_void, c_void, c_void, c_void, c_ip, c_ip, c_ip, c_int, c_int,
                                               c_int, c_int, c_float, c_int, c_int, c_int, c_void, c_void, c_ll, c_ip, c_void,
                                               c_void]
    self.lib.sb_experts_dense_bf16.restype = c_int
    self.lib.sb_graph_burst.argtypes = [c_void, c_void, c_void, c_ll, c_int, c_void, c_void, c_ll, c_void]
    self.lib.sb_graph_burst.restype = c_int
    self.lib.sb_stream_wait.argtypes = [c_void]
    self.lib.sb_stream_wait.restype = c_int
    self.lib.sb_sample_slices.argtypes = [c_int, c_int]
    self.lib.sb_sample_slices.restype = c_int

  def _stream(self):
    if self._step_stream is not None:
      return self._step_stream
    return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

  def hold_stream(self):
    """Context in which every launch goes to the stream that is current now, looked up once
    instead of once per launch (an engine step is a few hundred launches)."""
    return _HeldStream(self)

  def _library_product(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    """out = x . w^T through the matrix-product library with a kept algorithm; False when it
    has none for this shape."""
    stream = self._stream()
    workspace = self._library_workspaces.get(stream.value)
    if workspace is None:  # one per stream: products on different streams may run together
      workspace = self._library_workspaces[stream.value] = torch.empty(32 << 20, dtype=torch.uint8, device=self.device)
    m, k = x.shape
    rc = self.lib.sb_gemm_library_bf16(_ptr(x), _ptr(w), _ptr(out), m, w.shape[0], k, int(out.dtype == torch.float32),
                                       _ptr(workspace), workspace.numel(), stream)
    if rc > 0:
      raise KernelError(f"sb_gemm_library_bf16: cuBLAS status {rc}")
    self.launches += rc == 0
    return rc == 0

  def _library_head_products(self, x: torch.Tensor, x_head: int, w: torch.Tensor, out: torch.Tensor, out_head: int,
                             alpha: float) -> bool:
    """out[:, h * out_head : + N] = alpha * x[:, h * x_head : + K] . w[h]^T for w [H, N, K], all heads in one
    call of the matrix-product library (bfloat16); False when it does not take the shape."""
    if x.dtype != torch.bfloat16 or not self.direct_library_products:
      return False
    stream = self._stream()
    workspace = self._library_workspaces.get(stream.value)
    if workspace is None:
      workspace = self._library_workspaces[stream.value] = torch.empty(32 << 20, dtype=torch.uint8, device=self.device)
    h, n, k = w.shape
    rc = self.lib.sb_gemm_library_bf16_heads(_ptr(x), x.shape[1], x_head, _ptr(w), _ptr(out), out.shape[1], out_head,
                                             x.shape[0], h, n, k, float(alpha), _ptr(workspace), workspace.numel(), stream)
    if rc > 0:
      raise KernelError(f"sb_gemm_library_bf16_heads: cuBLAS status {rc}")
    self.launches += rc == 0
    return rc == 0

  def _call(self, name: str, *args) -> int:
    rc = getattr(self.lib, name)(*args, self._stream())
    self.launches += rc != -9  # -9: the kernel does not take the shape and launched nothing
    if rc != 0 and rc != -9:
      why = _STATUS.get(rc, f"CUDA error {rc}" if rc > 0 else f"status {rc}")
      raise KernelError(f"{name}: {why}")
    return rc

  def _new(self, *shape, dtype=None) -> torch.Tensor:
    return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)

  def check_errors(self) -> None:
    """Reads the device error word (synchronises); raises if a kernel refused an access."""
    word = int(self.err.item())
    if word:
      self.err.zero_()
      reasons = [msg for bit, msg in _ERRORS.items() if word & bit]
      raise KernelError("a kernel skipped an invalid access: " + "; ".join(reasons))

  # ---- checks ---------------------------------------------------------------
  def check_attention(self, head_dim: int, num_heads: int, num_kv_heads: int) -> None:
    """Refuses shapes no kernel takes; compiles the tensor-core kernels of this head size."""
    if head_dim <= 0 or head_dim % 2 or head_dim > 512:
      raise KernelError(f"attention kernels take even head sizes up to 512, got {head_dim}")
    if num_heads % num_kv_heads:
      raise KernelError(f"{num_heads} query heads are no multiple of {num_kv_heads} key/value heads")
    if self._uses_tensor_core_attention(head_dim, num_heads // num_kv_heads):
      self._attention_lib(head_dim)

  def _uses_tensor_core_attention(self, head_dim: int, group: int) -> bool:
    return (self.dtype == torch.bfloat16 and self.tensor_core_attention and head_dim % 16 == 0
            and head_dim <= 256 and group <= 64)  # a group must fit a 64-row tile

  def _attention_lib(self, head_dim: int):
    fns = self._attn_fns.get(head_dim)
    if fns is None:
      lib = build.load_attention(head_dim)
      c_int, c_float, c_void = ctypes.c_int, ctypes.c_float, ctypes.c_void_p
      prefill = getattr(lib, f"sb_attn_prefill_hd{head_dim}")
      prefill.argtypes = [c_void, c_void, c_void, c_int, c_void, c_void, c_void, c_int, c_int, c_int, c_int,
                          c_float, c_int, c_void, c_int, c_int, c_int, c_void, c_void]
      prefill.restype = c_int
      prefill_pooled = getattr(lib, f"sb_attn_prefill_pooled_hd{head_dim}")
      prefill_pooled.argtypes = prefill.argtypes[:-2] + [c_void, c_void, c_int, c_int, c_int, c_void, c_void]
      prefill_pooled.restype = c_int
      decode = getattr(lib, f"sb_attn_decode_hd{head_dim}")
      decode.argtypes = [c_void, c_void, c_void, c_int, c_void, c_void, c_void, c_void, c_int, c_int, c_int,
                         c_int, c_int, c_float, c_int, c_void, c_int, c_int, c_void, c_void, c_void, c_int,
                         c_void, c_void, c_int, c_void, c_int, c_void, c_void, c_void]
      decode.restype = c_int
      prefill_biased = getattr(lib, f"sb_attn_prefill_biased_hd{head_dim}")
      prefill_biased.argtypes = prefill.argtypes[:-2] + [c_void, c_void, c_void]
      prefill_biased.restype = c_int
      make_map = getattr(lib, f"sb_attn_tensor_map_hd{head_dim}")
      make_map.argtypes = [c_void, c_void, ctypes.c_longlong, c_int]
      make_map.restype = c_int
      prefill_tc = prefill_tc_biased = None
      if head_dim % 64 == 0:
        prefill_tc = getattr(lib, f"sb_attn_prefill_tc_hd{head_dim}")
        prefill_tc.argtypes = [c_void, c_void, c_void, c_int, c_void, c_void, c_void, c_int, c_int, c_int, c_int,
                               c_int, c_float, c_int, c_void, c_int, c_void, c_void]
        prefill_tc.restype = c_int
        prefill_tc_biased = getattr(lib, f"sb_attn_prefill_tc_biased_hd{head_dim}")
        prefill_tc_biased.argtypes = prefill_tc.argtypes[:-2] + [c_void, c_void, c_void]
        prefill_tc_biased.restype = c_int
      prefill_pair = None
      if head_dim in (128, 256):
        prefill_pair = getattr(lib, f"sb_attn_prefill_pair_hd{head_dim}")
        prefill_pair.argtypes = [c_void, c_void, c_void, c_int, c_void, c_void, c_void, c_int, c_int, c_int, c_int,
                                 c_int, c_float, c_int, c_void, c_int, c_void, c_void]
        prefill_pair.restype = c_int
      resident = getattr(lib, f"sb_attn_decode_resident_hd{head_dim}")
      resident.argtypes, resident.restype = [c_int], c_int
      slots = resident(1)
      if slots <= 0:
        raise KernelError(f"sb_attn_decode_resident: {_STATUS.get(slots, slots)}")
      self._decode_slots[head_dim] = slots
      fns = self._attn_fns[head_dim] = (prefill, decode, make_map, prefill_tc, prefill_pair, prefill_pooled,
                                        prefill_biased, prefill_tc_biased)
    return fns

  def _latent_fn(self, row_dim: int, value_dim: int):
    fn = self._latent_fns.get((row_dim, value_dim))
    if fn is None:
      lib = build.load_latent_attention(row_dim, value_dim)
      c_int, c_void = ctypes.c_int, ctypes.c_void_p
      fn = getattr(lib, f"sb_latent_attention_k{row_dim}_v{value_dim}")
      fn.argtypes = [c_void, c_void, c_void, c_int, c_void, c_void, c_void, c_void, c_int, c_int, c_int, c_int, c_int,
                     c_int, c_int, c_int, c_void, c_void, c_void, c_void]
      fn.restype = c_int
      self._latent_fns[(row_dim, value_dim)] = fn
    return fn

  def decode_chunk_for(self, kv_lo: Sequence[int], kv_hi: Sequence[int], num_kv_heads: int, head_dim: int) -> int:
    """Chunk length of split-key attention for sequences that see the keys [kv_lo, kv_hi).

    A work item is one chunk of one (sequence, kv head); the kernel's persistent grid draws items
    from a counter.  With `slots` resident blocks the launch lasts about
    ceil(items / slots) * (chunk + fixed cost of an item), so the chunk is the multiple of 64 that
    makes this smallest: the items then fill the grid in whole rounds instead of leaving most
    blocks idle in the last one.
    """
    if self.decode_chunk:
      return self.decode_chunk
    self._attention_lib(head_dim)
    slots = self._decode_slots[head_dim]
    lo, hi = np.asarray(kv_lo, dtype=np.int64), np.asarray(kv_hi, dtype=np.int64)
    # (From 128 keys: with 64 a lone sequence's window layers were 13 % slower than with 128,
    # although their items fit the grid either way: twice the items and twice the chunks to merge.)
    best, best_cost = 128, None
    for chunk in range(128, 2048 + 1, 64):
      items = int(((hi - 1) // chunk - lo // chunk + 1).sum()) * num_kv_heads
      cost = -(-items // slots) * (chunk + self.DECODE_ITEM_COST)
      if best_cost is None or cost <= best_cost:
        best, best_cost = chunk, cost
    return best

  # Fixed cost of a split-key work item (pipeline fill, partial result, its share of the merge),
  # in keys: about 2 microseconds of a block's share of the memory bandwidth.
  DECODE_ITEM_COST = 48

  @staticmethod
  def decode_chunk_range(q_start: np.ndarray, steps: int, window: int | None, chunk: int) -> tuple[np.ndarray, np.ndarray]:
    """First and last chunk index per sequence that a decode burst of `steps` steps touches: from
    the lowest key visible at the first step to the highest at the last."""
    qs = np.asarray(q_start, dtype=np.int64)
    lo = np.maximum(qs - window + 1, 0) // 64 * 64 if window else np.zeros_like(qs)
    return lo // chunk, (qs + steps - 1) // chunk

  @staticmethod
  def static_decode_plan(q_start: np.ndarray, steps: int, window: int | None, chunk: int,
                         items_per_seq: int) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Work list of the split-key kernel for a decode burst replayed from a CUDA graph.

    Every sequence gets exactly `items_per_seq` items, so the launch has a fixed size:
    the chunks that hold keys between the lowest key visible at the first step and the
    highest at the last step, then fillers (sequence -1).  A chunk that holds nothing
    visible at some step of the burst yields an empty partial result there.
    Returns (items [B * items_per_seq, 2], split_start [B], split_count [B]).
    """
    b = len(q_start)
    items = np.full((b, items_per_seq, 2), -1, dtype=np.int32)
    count = np.zeros(b, dtype=np.int32)
    firsts, lasts = CudaOps.decode_chunk_range(q_start, steps, window, chunk)
    for i, (first, last) in enumerate(zip(firsts.tolist(), lasts.tolist())):
      n = last - first + 1
      if n > items_per_seq:
        raise KernelError(f"decode burst needs {n} chunks per sequence, the graph holds {items_per_seq}")
      items[i, :n, 0] = i
      items[i, :n, 1] = np.arange(first, last + 1)
      count[i] = n
    start = (np.arange(b) * items_per_seq).astype(np.int32)
    return items.reshape(-1, 2), start, count

  def _tensor_map(self, storage: torch.Tensor, head_dim: int, page_size: int):
    """TMA descriptor of a cache storage (made once per storage), or None where TMA cannot be used."""
    if head_dim % 64 or page_size & (page_size - 1):
      return None
    # The descriptor holds the storage's address and its number of rows (rows beyond read as
    # zeros): another storage that the allocator puts at the same address must not find it.
    key = (storage.data_ptr(), storage.numel(), head_dim, page_size)
    buf = self._tensor_maps.get(key)
    if buf is None:
      make_map = self._attention_lib(head_dim)[2]
      buf = ctypes.create_string_buffer(128 + 64)
      aligned = (ctypes.addressof(buf) + 63) & ~63
      tile_keys = 32 if head_dim > 128 else 64
      rc = make_map(ctypes.c_void_p(aligned), _ptr(storage), storage.numel() // head_dim, min(page_size, tile_keys))
      buf = (buf, aligned if rc == 0 else None)
      self._tensor_maps[key] = buf
    return ctypes.c_void_p(buf[1]) if buf[1] is not None else None

  def _prefill_uses_tcgen05(self, head_dim: int, group: int, page_size: int) -> bool:
    return (self.prefill_tcgen05 and head_dim % 64 == 0 and 128 % group == 0
            and page_size & (page_size - 1) == 0)

  def _prefill_uses_pairs(self, head_dim: int, group: int, page_size: int) -> bool:
    """The tcgen05 prefill kernel by pairs of blocks (csrc/attention_tc_pair.cu)."""
    return (self.prefill_pairs and self._prefill_uses_tcgen05(head_dim, group, page_size)
            and head_dim in (128, 256) and page_size >= 64)

  def _prefill_rows(self, head_dim: int, group: int, page_size: int) -> int:
    """Query rows of a prefill work item: 256 for a pair of blocks, 128 for the tcgen05 kernel, else the mma.sync tile."""
    if self._prefill_uses_pairs(head_dim, group, page_size):
      return 256
    if self._prefill_uses_tcgen05(head_dim, group, page_size):
      return 128
    return self.prefill_rows or 64

  def _plan_key(self, window: int | None, group: int, num_kv_heads: int, head_dim: int, page_size: int) -> tuple:
    """Where a step keeps the work lists of one kind of attention layer in `ctx.memo`.  Layers
    share lists only if everything the lists are cut for agrees: the window, the group, the
    number of kv heads and the head size (they set the chunk length) and the rows of a prefill tile."""
    return ("attention_plan", window, group, num_kv_heads, head_dim, self._prefill_rows(head_dim, group, page_size))

  def attention_graph_plan(self, *, window: int | None, num_heads: int, num_kv_heads: int, head_dim: int,
                           batch: int, bucket: int, max_burst: int, page_size: int):
    """The static work list a decode graph needs for one kind of attention layer, or None when
    the kernel that serves it reads no list (the general kernel)."""
    group = num_heads // num_kv_heads
    if not self._uses_tensor_core_attention(head_dim, group):
      return None
    return AttentionGraphPlan(self, window, group, num_kv_heads, head_dim, batch, bucket, max_burst, page_size)

  def pooled_attention_graph_plan(self, *, window: int | None, num_heads: int, num_kv_heads: int, head_dim: int,
                                  value_dim: int, pool: int, batch: int, page_size: int):
    """The static work list a decode graph needs for a layer with pooled blocks, or None when the
    general kernel serves it (which reads no list)."""
    group = num_heads // num_kv_heads
    if value_dim != head_dim or not window or not self._uses_tensor_core_attention(head_dim, group):
      return None
    return PooledAttentionGraphPlan(self._plan_key(window, group, num_kv_heads, head_dim, page_size) + ("pooled", pool), batch)

  def _attention_plan(self, ctx: Any, window: int | None, group: int, force_rows: int = 0,
                      num_kv_heads: int = 1, head_dim: int = 0, tag: tuple = (), all_tiles: bool = False) -> dict:
    """Work lists of the two tensor-core kernels for this step, per kind of layer (`_plan_key`).

    Sequences with at most 16 query rows per kv head (one or a few new tokens) go to the
    split-key kernel: their keys are cut into chunks at multiples of `chunk` of the
    absolute position, one work item per chunk.  The others are cut into tiles of
    64 // group or 128 // group tokens for the prefill kernel, heaviest tile first.
    """
    key = self._plan_key(window, group, num_kv_heads, head_dim, ctx.page_size) + tag
    plan = ctx.memo.get(key)
    if plan is not None:
      return plan
    cu_q, q_start = ctx.host["cu_q"], ctx.host["q_start"].astype(np.int64)
    q_len = np.diff(cu_q).astype(np.int64)
    small = (q_len * group <= 16) & (not all_tiles)  # all_tiles: the tile kernel takes every sequence
    # Tiles of 64 query rows (finer grains balance better over the SMs than tiles of 128).
    rows_per_tile = force_rows or self.prefill_rows or 64
    tokens_per_tile = rows_per_tile // group
    num_seqs = len(q_len)
    pre = []
    for b in np.nonzero(~small)[0]:
      for i0 in range(0, int(q_len[b]), tokens_per_tile):
        last = int(q_start[b]) + min(i0 + tokens_per_tile, int(q_len[b]))
        first = max(int(q_start[b]) + i0 - window + 1, 0) if window else 0
        pre.append((last - first, int(b), i0))
    pre.sort(key=lambda x: -x[0])
    if force_rows in (128, 256):
      # The tcgen05 kernels' blocks, one per (tile of queries, kv head), longest walk first over all
      # heads: the GPU holds 74 pairs (or 148 single blocks) at once and gives the next one in the list to the SMs that
      # are free first, so this order fills them evenly (listed head by head, 128 blocks of a
      # 4,096-token prompt ended as late as 53 tiles' time where 37 are enough).
      prefill_items = np.array([(b, i0, m) for _, b, i0 in pre for m in range(num_kv_heads)],
                               dtype=np.int32).reshape(-1, 3)
    else:
      prefill_items = np.array([(b, i0) for _, b, i0 in pre], dtype=np.int32).reshape(-1, 2)
    kv_hi = q_start + q_len
    kv_lo = np.maximum(q_start - window + 1, 0) if window else np.zeros_like(q_start)
    kv_lo = kv_lo // 64 * 64
    dec = np.nonzero(small)[0]
    chunk = 64
    if len(dec):
      chunk = self.decode_chunk_for(kv_lo[dec], kv_hi[dec], num_kv_heads, head_dim)
    split_start = np.zeros(num_seqs, dtype=np.int32)
    split_count = np.zeros(num_seqs, dtype=np.int32)
    dec_items = []
    for b in dec:
      first, last = int(kv_lo[b]) // chunk, (int(kv_hi[b]) - 1) // chunk
      split_start[b] = len(dec_items)
      split_count[b] = last - first + 1
      dec_items += [(int(b), c) for c in range(first, last + 1)]
    decode_items = np.array(dec_items, dtype=np.int32).reshape(-1, 2)
    flat = np.concatenate([prefill_items.reshape(-1), decode_items.reshape(-1), split_start, split_count])
    dev = torch.from_numpy(flat).to(self.device, non_blocking=True)
    n_pre, n_dec = prefill_items.size, decode_items.size
    plan = dict(
        num_prefill=len(prefill_items), num_decode=len(decode_items), chunk=chunk, rows_per_tile=rows_per_tile,
        item_width=prefill_items.shape[1], rows_max=int((q_len[dec] * group).max()) if len(dec) else 0,
        prefill_items=dev[:n_pre], decode_items=dev[n_pre:n_pre + n_dec],
        split_start=dev[n_pre + n_dec:n_pre + n_dec + num_seqs], split_count=dev[n_pre + n_dec + num_seqs:])
    ctx.memo[key] = plan
    return plan

  # ---- dense ----------------------------------------------------------------
  def embed(self, table: torch.Tensor, ids: torch.Tensor, scale: float, positions: torch.Tensor | None = None,
            position_table: torch.Tensor | None = None, round_scale: bool = True) -> torch.Tensor:
    """float32 rows table[id] * scale (+ position_table[position]).  `round_scale`: the factor is
    rounded to the table's dtype first."""
    if position_table is not None or not round_scale:
      if position_table is not None and position_table.dtype != table.dtype:
        raise KernelError("the embedding table and the position table must share one dtype")
      out = self._new(ids.numel(), table.shape[1], dtype=torch.float32)
      self._call("sb_embed_positions", _ptr(table), _ptr(position_table), _code(table), _ptr(ids), _ptr(positions),
                 float(scale), _ptr(out), ids.numel(), table.shape[1], table.shape[0],
                 position_table.shape[0] if position_table is not None else 0, _ptr(self.err))
      return out
    if table.dtype == torch.bfloat16:
      # The reference rounds the constant to the activation dtype (simply/utils/module.py:477-481).
      rounded = self._rounded_scales.get(scale)
      if rounded is None:
        rounded = self._rounded_scales[scale] = float(torch.tensor(scale, dtype=torch.float32).to(torch.bfloat16))
      scale = rounded
    out = self._new(ids.numel(), table.shape[1], dtype=torch.float32)
    self._call("sb_embed", _ptr(table), _code(table), _ptr(ids), float(scale), _ptr(out), ids.numel(),
               table.shape[1], table.shape[0], _ptr(self.err))
    return out

  def cast(self, x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if x.dtype == dtype:
      return x
    out = self._new(*x.shape, dtype=dtype)
    self._call("sb_cast", _ptr(x), _code(x), _ptr(out), _code(out), x.numel())
    return out

  def _mid_product(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, cap: float = 0.0,
                   activation: int = 0, split: int | None = None) -> bool:
    """The weight-streaming product for a serving batch (17 to 128 tokens); False when it does
    not take the shape."""
    m, k = x.shape
    n = w.shape[0]
    split = self.mid_split if split is None else split
    return self._call("sb_gemm_stream_tc", _ptr(x), _ptr(w), _ptr(out), m, n, k, epilogue, float(cap), activation,
                      split, self.mid_stages, _ptr(self.err)) == 0

  def linear(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [M, K] . w[N, K]^T -> [M, N] in the activation dtype."""
    m, k = x.shape
    n = w.shape[0]
    if w.dtype == torch.float32:
      # Float32 weights (the 32-bit path, or a tensor stored in 32 bits): true float32 product.
      xf = self.cast(x, torch.float32)
      out = self._new(m, n, dtype=torch.float32)
      self._call("sb_gemm_f32_nt", _ptr(xf), _ptr(w), _ptr(out), m, n, k, 0.0)
      return self.cast(out, self.dtype)
    x = self.cast(x, torch.bfloat16)
    if m <= self.skinny_max_rows:
      out = self._new(m, n, dtype=torch.bfloat16)
      if self._call("sb_gemm_skinny_bf16", _ptr(x), _ptr(w), _ptr(out), m, n, k, 0, 0.0, 0, self.skinny_warps) == 0:
        return out
    elif m <= self.mid_rows["plain"] and self.mid_rows_kernel and x.is_contiguous() and w.is_contiguous():
      out = self._new(m, n, dtype=torch.bfloat16)
      if self._mid_product(x, w, out, 0):
        return out
    if self.direct_library_products and x.is_contiguous() and w.is_contiguous():
      out = self._new(m, n, dtype=torch.bfloat16)
      if self._library_product(x, w, out):
        return out
    return torch.mm(x, w.t())

  def gated_linear(self, x: torch.Tensor, w_gate_up: torch.Tensor, activation: int, limit: float = 0.0) -> torch.Tensor:
    """act(x . w_gate^T) * (x . w_up^T) with w_gate_up = [gate rows; up rows]: [M, N/2].  Activation 3
    (clamped) takes `limit` and acts on both halves (csrc/elementwise.cu)."""
    m, k = x.shape
    n = w_gate_up.shape[0]
    if w_gate_up.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and m <= self.skinny_max_rows:
      out = self._new(m, n // 2, dtype=torch.bfloat16)
      if self._call("sb_gemm_skinny_bf16", _ptr(x), _ptr(w_gate_up), _ptr(out), m, n, k, 2, float(limit),
                    activation, self.skinny_warps) == 0:
        return out
    if (w_gate_up.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and self.mid_rows_kernel
        and self.skinny_max_rows < m <= self.mid_rows["gated"] and x.is_contiguous() and w_gate_up.is_contiguous()):
      out = self._new(m, n // 2, dtype=torch.bfloat16)
      if self._mid_product(x, w_gate_up, out, 2, cap=limit, activation=activation):
        return out
    if (w_gate_up.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and m >= self.gated_tc_min_rows > 0
        and x.is_contiguous() and w_gate_up.is_contiguous()):
      out = self._new(m, n // 2, dtype=torch.bfloat16)
      if self._call("sb_gemm_gated_tc", _ptr(x), _ptr(w_gate_up), _ptr(out), m, n // 2, k, activation, float(limit),
                    self.gated_tc_blocks, int(self.gated_tc_pairs), _ptr(self.err)) == 0:
        return out
    return self.gated_activation(self.linear(x, w_gate_up), activation, limit)

  def lm_head(self, x: torch.Tensor, table: torch.Tensor, cap: float, scale: float = 1.0) -> torch.Tensor:
    """float32 logits [R, vocab] = softcap(scale * x . table^T)."""
    if scale != 1.0:
      out = self.lm_head(x, table, 0.0)
      self._call("sb_scale_values", _ptr(out), float(scale), out.numel())
      if cap:
        self._call("sb_soft_cap", _ptr(out), float(cap), out.numel())
      return out
    r, k = x.shape
    v = table.shape[0]
    out = self._new(r, v, dtype=torch.float32)
    if table.dtype == torch.float32:
      xf = self.cast(x, torch.float32)
      self._call("sb_gemm_f32_nt", _ptr(xf), _ptr(table), _ptr(out), r, v, k, float(cap))
      return out
    x = self.cast(x, torch.bfloat16)
    chunk = 32
    if chunk < r <= self.mid_rows["head"] and self.mid_rows_kernel and k % 8 == 0 and x.is_contiguous():
      # 33 to 128 rows: one pass over the table instead of several
      if self._mid_product(x, table, out, 1, cap=cap, split=1):
        return out
    if r > chunk and k % 8 == 0:
      if self.direct_library_products and x.is_contiguous() and self._library_product(x, table, out):
        self._call("sb_soft_cap", _ptr(out), float(cap), out.numel())
        return out
      try:
        torch.mm(x, table.t(), out_dtype=torch.float32, out=out)
        self._call("sb_soft_cap", _ptr(out), float(cap), out.numel())
        return out
      except (TypeError, RuntimeError):
        pass
    if k % 8:
      # A width without whole 16-byte groups: the float32 product on a float32 copy of the table.
      key = (table.data_ptr(), tuple(table.shape))
      wide = self._wide_tables.get(key)
      if wide is None:
        wide = self._wide_tables[key] = table.float().contiguous()
      self._call("sb_gemm_f32_nt", _ptr(self.cast(x, torch.float32)), _ptr(wide), _ptr(out), r, v, k, float(cap))
      return out
    for r0 in range(0, r, chunk):
      rows = min(chunk, r - r0)
      self._call("sb_gemm_skinny_bf16", _ptr(x[r0:]), _ptr(table), _ptr(out[r0:]), rows, v, k, 1,
                 float(cap), 0, self.skinny_warps)
    return out

  def gated_activation(self, gate_up: torch.Tensor, activation: int, limit: float = 0.0) -> torch.Tensor:
    t, two_f = gate_up.shape
    out = self._new(t, two_f // 2, dtype=gate_up.dtype)
    self._call("sb_gated_activation", _ptr(gate_up), _code(gate_up), _ptr(out), t, two_f // 2, activation,
               float(limit))
    return out

  # ---- norms ----------------------------------------------------------------
  def rms_norm(self, x: torch.Tensor, w: torch.Tensor, eps: float, plus_one: bool) -> torch.Tensor:
    out = self._new(*x.shape)
    self._call("sb_rms_norm", _ptr(x), _code(x), _ptr(w), int(w.dtype == torch.float32), float(eps),
               int(plus_one), _ptr(out), _code(out), x.shape[0], x.shape[1])
    return out

  def residual_norm(self, h: torch.Tensor, branch: torch.Tensor | None, post: Any, pre: Any,
                    rows: torch.Tensor | None, branch2: torch.Tensor | None = None) -> torch.Tensor | None:
    """h += norm_post(branch) (+ branch2, as it is); returns norm_pre(h) in the activation dtype (see
    csrc/elementwise.cu)."""
    width = h.shape[1]
    num_rows = h.shape[0] if rows is None else rows.numel()
    y = self._new(num_rows, width) if pre is not None else None
    if branch is None and pre is None:
      return None
    if branch is not None and branch.dtype != self.dtype:
      branch = self.cast(branch, self.dtype)
    if branch2 is not None and branch2.dtype != self.dtype:
      branch2 = self.cast(branch2, self.dtype)
    if branch2 is not None and branch is None:
      branch, branch2 = branch2, None
    wp, wq = (post.weight if post is not None else None), (pre.weight if pre is not None else None)
    self._call(
        "sb_residual_norm", _ptr(h), _ptr(branch), _ptr(branch2), _BF16 if self.dtype == torch.bfloat16 else _F32,
        _ptr(wp), int(wp is not None and wp.dtype == torch.float32),
        float(post.eps) if post is not None else 0.0, int(post.plus_one) if post is not None else 0,
        _ptr(wq), int(wq is not None and wq.dtype == torch.float32),
        float(pre.eps) if pre is not None else 0.0, int(pre.plus_one) if pre is not None else 0,
        _ptr(rows), _ptr(y), num_rows, width, h.shape[0], _ptr(self.err))
    return y

  def gather_rows(self, x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    out = self._new(rows.numel(), x.shape[1], dtype=x.dtype)
    self._call("sb_gather_rows", _ptr(x), _code(x), _ptr(rows), _ptr(out), rows.numel(), x.shape[1],
               x.shape[0], _ptr(self.err))
    return out

  def add_to_residual(self, h: torch.Tensor, x: torch.Tensor) -> None:
    self._call("sb_add_to_residual", _ptr(h), _ptr(x), _code(x), h.numel())

  # ---- a stream whose norm computes no statistics ------------------------------------------
  def scaled_residual_tanh(self, h: torch.Tensor, branch: torch.Tensor | None, scale: torch.Tensor | None,
                           branch2: torch.Tensor | None, scale2: torch.Tensor | None, pre: Any,
                           rows: torch.Tensor | None) -> torch.Tensor | None:
    """h += scale * branch + scale2 * branch2 (float32 [width] factors; None: the branch as it is);
    returns tanh(alpha h) w + b for the norm `pre` (its float32 `alpha` [1], `weight`, `bias`) in the
    activation dtype, or None without one.  With `rows` only those rows are computed and h is left
    as it is (csrc/stream_pointwise.cu)."""
    if h.dtype != torch.float32:
      h = self.cast(h, torch.float32)
    width = h.shape[1]
    if branch is None and branch2 is not None:
      branch, scale, branch2, scale2 = branch2, scale2, None, None
    if branch is None and pre is None:
      return None
    if branch is not None and branch.dtype != self.dtype:
      branch = self.cast(branch, self.dtype)
    if branch2 is not None and branch2.dtype != self.dtype:
      branch2 = self.cast(branch2, self.dtype)
    num_rows = h.shape[0] if rows is None else rows.numel()
    y = self._new(num_rows, width) if pre is not None else None
    self._call("sb_scaled_residual_tanh", _ptr(h), _ptr(branch), _ptr(scale), _ptr(branch2), _ptr(scale2),
               _BF16 if self.dtype == torch.bfloat16 else _F32, _ptr(pre.alpha) if pre is not None else None,
               _ptr(pre.weight) if pre is not None else None, _ptr(pre.bias) if pre is not None else None,
               _ptr(rows), _ptr(y), num_rows, width, h.shape[0], _ptr(self.err))
    return y

  def scale_channels(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x * w with a float32 factor per channel, in the activation dtype."""
    h = torch.zeros(x.shape, dtype=torch.float32, device=self.device)
    self.scaled_residual_tanh(h, x, w, None, None, None, None)
    return self.cast(h, self.dtype)

  def pack_pair(self, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """[a, b] side by side, float32 [T, W] each, as [T, 2 W] in the activation dtype."""
    out = self._new(a.shape[0], 2 * a.shape[1])
    self._call("sb_pack_pair", _ptr(a), _ptr(b), _ptr(out), _code(out), a.shape[0], a.shape[1])
    return out

  def linear_wide(self, x: torch.Tensor, w: torch.Tensor, row: torch.Tensor | None = None) -> torch.Tensor:
    """x . w^T (+ row) with float32 sums left as they are: float32 [M, N]."""
    out = self.lm_head(x, w, 0.0)
    if row is not None:
      self._call("sb_add_row", _ptr(out), _ptr(row), out.shape[0], out.shape[1])
    return out

  def linear_xielu(self, x: torch.Tensor, w: torch.Tensor, act: torch.Tensor,
                   factors: tuple[float, float] | None = None) -> torch.Tensor:
    """xielu(x . w^T) with the activation's two learned numbers `act` (float32 [2]).  `factors`:
    (softplus(act[0]), 1/2 + softplus(act[1])) as the host knows them; with them a step of few
    tokens activates on the product's sums (csrc/gemm_skinny_bf16.cu)."""
    m, k = x.shape
    if (factors is not None and w.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
        and m <= self.skinny_max_rows):
      out = self._new(m, w.shape[0], dtype=torch.bfloat16)
      if self._call("sb_gemm_skinny_bf16_xielu", _ptr(x), _ptr(w), _ptr(out), m, w.shape[0], k, float(factors[0]),
                    float(factors[1]), self.skinny_warps) == 0:
        return out
    z = self.linear(x, w)
    self._call("sb_xielu", _ptr(z), _ptr(act), _ptr(z), _code(z), z.numel())
    return z

  # ---- positions ------------------------------------------------------------
  def rotation_tables(self, positions: torch.Tensor, timescale: torch.Tensor, scale_factor: float):
    t, half = positions.numel(), timescale.numel()
    cos = self._new(t, half, dtype=torch.float32)
    sin = self._new(t, half, dtype=torch.float32)
    self._call("sb_rotation_tables", _ptr(positions), _ptr(timescale), float(scale_factor), _ptr(cos),
               _ptr(sin), t, half)
    return cos, sin

  def rope_and_cache_write(self, qkv: torch.Tensor, tables, q_scale: float, num_heads: int,
                           num_kv_heads: int, head_dim: int, storage: torch.Tensor | None,
                           block_table: torch.Tensor, ctx: Any) -> torch.Tensor:
    t = qkv.shape[0]
    q = self._new(t, num_heads, head_dim, dtype=qkv.dtype)
    cos, sin = tables if tables is not None else (None, None)
    if storage is not None and storage.dtype != qkv.dtype:
      raise KernelError("cache and activations must share one dtype")
    self._call("sb_rope_cache_write", _ptr(qkv), _code(qkv), _ptr(cos), _ptr(sin), float(q_scale), _ptr(q),
               _ptr(storage), _ptr(block_table), block_table.shape[1], _ptr(ctx.token_seq),
               _ptr(ctx.positions), t, num_heads, num_kv_heads, head_dim, ctx.page_size,
               storage.shape[0] if storage is not None else 0, int(storage is not None), _ptr(self.err))
    return q

  def project_rotate_store(self, x: torch.Tensor, w_qkv: torch.Tensor, tables, q_scale: float, num_heads: int,
                           num_kv_heads: int, head_dim: int, storage: torch.Tensor | None,
                           block_table: torch.Tensor, ctx: Any) -> torch.Tensor:
    """The fused q, k, v projection, then rotation, query scale and the stores: queries
    [T, num_heads, head_dim] are returned, keys and values go into the pages of `storage`.

    Steps of a few tokens do it in one kernel (the product's epilogue rotates and stores);
    larger ones as a product followed by `rope_and_cache_write`.
    """
    t, k = x.shape
    if (self.fused_qkv_rope and self.dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16
        and t <= self.skinny_max_rows and t <= 16 and head_dim % 32 == 0 and k % 8 == 0):
      x = self.cast(x, torch.bfloat16)
      q = self._new(t, num_heads, head_dim, dtype=torch.bfloat16)
      cos, sin = tables if tables is not None else (None, None)
      if storage is not None and storage.dtype != torch.bfloat16:
        raise KernelError("cache and activations must share one dtype")
      rc = self._call("sb_qkv_rope_skinny", _ptr(x), _ptr(w_qkv), t, k, _ptr(cos), _ptr(sin), float(q_scale),
                      _ptr(q), _ptr(storage), _ptr(block_table), block_table.shape[1], _ptr(ctx.token_seq),
                      _ptr(ctx.positions), num_heads, num_kv_heads, head_dim, ctx.page_size,
                      storage.shape[0] if storage is not None else 0, _ptr(self.err), self.skinny_warps)
      if rc == 0:
        return q
    if (self.fused_qkv_rope and self.mid_rows_kernel and self.dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16
        and self.skinny_max_rows < t <= self.mid_rows["qkv"] and head_dim % 128 == 0 and k % 8 == 0):
      x = self.cast(x, torch.bfloat16)
      q = self._new(t, num_heads, head_dim, dtype=torch.bfloat16)
      cos, sin = tables if tables is not None else (None, None)
      if storage is not None and storage.dtype != torch.bfloat16:
        raise KernelError("cache and activations must share one dtype")
      args = (_ptr(x), _ptr(w_qkv), t, k, _ptr(cos), _ptr(sin), float(q_scale),
              _ptr(q), _ptr(storage), _ptr(block_table), block_table.shape[1], _ptr(ctx.token_seq),
              _ptr(ctx.positions), num_heads, num_kv_heads, head_dim, ctx.page_size,
              storage.shape[0] if storage is not None else 0, _ptr(self.err), self.mid_split)
      rc = self._call("sb_qkv_rope_stream_tc", *args, self.mid_stages)
      if rc == 0:
        return q
    qkv = self.linear(x, w_qkv)
    return self.rope_and_cache_write(qkv, tables, q_scale, num_heads, num_kv_heads, head_dim, storage,
                                     block_table, ctx)

  # ---- attention ------------------------------------------------------------
  def paged_attention(self, q: torch.Tensor, storage: torch.Tensor, block_table: torch.Tensor, ctx: Any, *,
                      num_heads: int, num_kv_heads: int, head_dim: int, logit_softcap: float,
                      window: int | None, value_dim: int | None = None, pooled: tuple | None = None,
                      values_in_keys: bool = False, sink: torch.Tensor | None = None,
                      distance_bias: torch.Tensor | None = None) -> torch.Tensor:
    """`value_dim`: size of a value head where it is not the key heads'.  `pooled`: (storage of block
    entries, its block table, block length): with a window, one key and value per whole block that
    has left the window, under the same softmax.  `values_in_keys`: an entry's value is the first
    `value_dim` numbers of its key row (a cache of latents).  `sink`: float32 [heads], a number per
    head whose exponential joins the softmax's denominator (csrc/attention_generic.cu).
    `distance_bias`: float32 [2, heads], r1 and r2 per head: the score of query i and key j loses
    r1 log(1 + r2 (i - j))."""
    t = q.shape[0]
    value_dim = head_dim if value_dim is None else value_dim
    out = self._new(t, num_heads * value_dim, dtype=q.dtype)
    group = num_heads // num_kv_heads
    if (values_in_keys or sink is not None) and (logit_softcap or pooled is not None):
      raise KernelError("latent rows and sinks go with neither a score cap nor pooled blocks")
    if distance_bias is not None and (pooled is not None or values_in_keys):
      raise KernelError("a distance bias goes with neither pooled blocks nor latent rows")
    # (a distance bias with key size = value size in bfloat16: the mma.sync tile kernels below)
    biased_on_tensor_cores = (distance_bias is not None and value_dim == head_dim and q.dtype == torch.bfloat16
                              and self._uses_tensor_core_attention(head_dim, group))
    if (pooled is not None or value_dim != head_dim or values_in_keys or sink is not None
        or (distance_bias is not None and not biased_on_tensor_cores)):
      pool, pool_table, pool_len = pooled if pooled is not None else (None, None, 0)
      if pool is not None and pool.dtype != storage.dtype:
        raise KernelError("block entries and the cache must share one dtype")
      pool_args = (_ptr(pool), _ptr(pool_table), pool_table.shape[1] if pool is not None else 0, int(pool_len),
                   pool.shape[0] if pool is not None else 0)

      def general():
        self._call("sb_paged_attention_general", _ptr(q), _code(q), _ptr(storage), _ptr(block_table),
                   block_table.shape[1], _ptr(ctx.token_seq), _ptr(ctx.positions), _ptr(out), t, num_heads,
                   num_kv_heads, head_dim, value_dim, ctx.page_size, storage.shape[0], float(logit_softcap),
                   int(window or 0), *pool_args, int(values_in_keys), _ptr(sink), _ptr(distance_bias), _ptr(self.err))

      # bfloat16 with key size = value size: the tensor-core tile kernel (mma.sync tiles of 64 rows,
      # the block entries in tiles of their own ahead of the tokens) for prompt portions and single
      # tokens alike; other shapes and float32: the general kernel.
      if (values_in_keys and pooled is None and num_kv_heads == 1 and q.dtype == torch.bfloat16
          and self.tensor_core_attention and build.latent_shape_ok(head_dim, value_dim)):
        # a cache of latents in bfloat16: the tensor-core kernel of this shape (csrc/attention_latent_mma.cu)
        # Steps of few rows per sequence (single tokens): every sequence's keys are split over several
        # blocks, by what a sequence can hold (not by what it holds now: a captured graph keeps the launch).
        splits, part_ml, part_o = 1, None, None
        if ctx.max_q_len * num_heads <= 32 and t * num_heads <= 8192:
          reach = min(int(window or (1 << 30)), block_table.shape[1] * ctx.page_size)
          splits = max(1, min(16, reach // 128))
        if splits > 1:
          part_ml = self._new(t * num_heads * splits * 2, dtype=torch.float32)
          part_o = self._new(t * num_heads * splits * value_dim, dtype=torch.float32)
        rc = self._latent_fn(head_dim, value_dim)(
            _ptr(q), _ptr(storage), _ptr(block_table), block_table.shape[1], _ptr(ctx.cu_q), _ptr(ctx.q_start),
            _ptr(out), _ptr(sink), t, ctx.num_seqs, ctx.max_q_len, num_heads, ctx.page_size, storage.shape[0],
            int(window or 0), splits, _ptr(part_ml), _ptr(part_o), _ptr(self.err), self._stream())
        self.launches += 1 + (splits > 1)
        if rc:
          raise KernelError(f"sb_latent_attention: {_STATUS.get(rc, rc)}")
        return out
      tensor_cores = (pooled is not None and value_dim == head_dim and q.dtype == torch.bfloat16 and window
                      and self._uses_tensor_core_attention(head_dim, group))
      if not tensor_cores:
        general()
        return out
      key = self._plan_key(window, group, num_kv_heads, head_dim, ctx.page_size) + ("pooled", pool_len)
      plan = ctx.memo.get(key)  # (a decode graph brings its static list)
      if plan is None:
        plan = self._attention_plan(ctx, window, group, 0, num_kv_heads, head_dim, tag=("pooled", pool_len),
                                    all_tiles=True)
      if plan["num_prefill"]:
        rc = self._attention_lib(head_dim)[5](
            _ptr(q), _ptr(storage), _ptr(block_table), block_table.shape[1], _ptr(ctx.cu_q), _ptr(ctx.q_start),
            _ptr(out), num_heads, num_kv_heads, ctx.page_size, storage.shape[0], float(logit_softcap), int(window),
            _ptr(plan["prefill_items"]), plan["num_prefill"], plan["rows_per_tile"], int(self.prefill_single_key_group),
            *pool_args, _ptr(self.err), self._stream())
        self.launches += 1
        if rc:
          raise KernelError(f"sb_attn_prefill_pooled: {_STATUS.get(rc, rc)}")
      return out
    if q.dtype == torch.bfloat16 and self._uses_tensor_core_attention(head_dim, group):
      prefill, decode, _, prefill_tc, prefill_pair = self._attention_lib(head_dim)[:5]
      # A distance bias: the tcgen05 kernel by single blocks where it takes the shape (no cap beside
      # it), else the mma.sync tile kernel; not the kernel by pairs.
      use_tc = (prefill_tc is not None and self._prefill_uses_tcgen05(head_dim, group, ctx.page_size)
                and (distance_bias is None or not logit_softcap))
      use_pair = (prefill_pair is not None and self._prefill_uses_pairs(head_dim, group, ctx.page_size)
                  and distance_bias is None)
      plan = self._attention_plan(ctx, window, group, 256 if use_pair else (128 if use_tc else 0), num_kv_heads, head_dim)
      common = (_ptr(q), _ptr(storage), _ptr(block_table), block_table.shape[1], _ptr(ctx.cu_q),
                _ptr(ctx.q_start))
      sizes = (num_heads, num_kv_heads, ctx.page_size, storage.shape[0], float(logit_softcap), int(window or 0))
      if plan["num_prefill"] and use_pair:
        rc = prefill_pair(*common, _ptr(out), t, *sizes, _ptr(plan["prefill_items"]), plan["num_prefill"],
                          _ptr(self.err), self._stream())
        self.launches += 1
        if rc:
          raise KernelError(f"sb_attn_prefill_pair: {_STATUS.get(rc, rc)}")
      elif plan["num_prefill"] and use_tc and distance_bias is not None:
        tiles = plan
        if plan["rows_per_tile"] != 128 or plan.get("item_width") != 3:  # (a list cut for another kernel)
          tiles = self._attention_plan(ctx, window, group, 128, num_kv_heads, head_dim, tag=("rows", 128))
        rc = self._attention_lib(head_dim)[7](*common, _ptr(out), t, *sizes, _ptr(tiles["prefill_items"]),
                                              tiles["num_prefill"], _ptr(distance_bias), _ptr(self.err), self._stream())
        self.launches += 1
        if rc:
          raise KernelError(f"sb_attn_prefill_tc_biased: {_STATUS.get(rc, rc)}")
      elif plan["num_prefill"] and use_tc:
        rc = prefill_tc(*common, _ptr(out), t, *sizes, _ptr(plan["prefill_items"]), plan["num_prefill"],
                        _ptr(self.err), self._stream())
        self.launches += 1
        if rc:
          raise KernelError(f"sb_attn_prefill_tc: {_STATUS.get(rc, rc)}")
      elif plan["num_prefill"] and distance_bias is not None:
        tiles = plan
        if plan.get("item_width", 2) != 2:  # (a list cut for the tcgen05 kernels, made by a layer without a bias)
          tiles = self._attention_plan(ctx, window, group, 64, num_kv_heads, head_dim, tag=("rows", 64))
        rc = self._attention_lib(head_dim)[6](
            *common, _ptr(out), *sizes, _ptr(tiles["prefill_items"]), tiles["num_prefill"], tiles["rows_per_tile"],
            int(self.prefill_single_key_group), _ptr(distance_bias), _ptr(self.err), self._stream())
        self.launches += 1
        if rc:
          raise KernelError(f"sb_attn_prefill_biased: {_STATUS.get(rc, rc)}")
      elif plan["num_prefill"]:
        rc = prefill(*common, _ptr(out), *sizes, _ptr(plan["prefill_items"]), plan["num_prefill"],
                     plan["rows_per_tile"], int(self.prefill_single_key_group), _ptr(self.err), self._stream())
        self.launches += 1
        if rc:
          raise KernelError(f"sb_attn_prefill: {_STATUS.get(rc, rc)}")
      if plan["num_decode"]:
        n = plan["num_decode"] * num_kv_heads * plan["rows_max"]
        part_o = self._new(n * head_dim, dtype=torch.float32)
        part_ml = self._new(n * 2, dtype=torch.float32)
        rc = decode(*common, _ptr(ctx.token_seq), _ptr(out), t, *sizes, _ptr(plan["decode_items"]),
                    plan["num_decode"], plan["chunk"], _ptr(part_o), _ptr(part_ml), _ptr(self._attn_counter),
                    plan["rows_max"],
                    _ptr(plan["split_start"]), _ptr(plan["split_count"]), self.decode_variant,
                    self._tensor_map(storage, head_dim, ctx.page_size),
                    int(getattr(ctx, "older_keys_settled", False)), _ptr(distance_bias), _ptr(self.err), self._stream())
        self.launches += 2
        if rc:
          raise KernelError(f"sb_attn_decode: {_STATUS.get(rc, rc)}")
      return out
    self._call("sb_paged_attention_generic", _ptr(q), _code(q), _ptr(storage), _ptr(block_table),
               block_table.shape[1], _ptr(ctx.token_seq), _ptr(ctx.positions), _ptr(out), t, num_heads,
               num_kv_heads, head_dim, ctx.page_size, storage.shape[0], float(logit_softcap),
               int(window or 0), _ptr(self.err))
    return out

  # ---- attention with normed queries and keys ---------------------------------
  def qk_norm_rotate_store(self, qkv: torch.Tensor, q_norm: torch.Tensor, k_norm: torch.Tensor | None, eps: float,
                           head_scale: torch.Tensor, rot_freq: torch.Tensor | None, value_freq: torch.Tensor | None,
                           num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int,
                           storage: torch.Tensor | None, block_table: torch.Tensor, ctx: Any) -> torch.Tensor:
    """qkv [T, q | k | v] -> queries [T, num_heads, head_dim], normed over the whole projection,
    rotated and scaled per head; keys (normed, rotated) and values (rotated with `value_freq`) go
    into the pages of `storage` (csrc/attention_prepare.cu).  `num_kv_heads = 0`: queries only."""
    t = qkv.shape[0]
    q = self._new(t, num_heads, head_dim, dtype=qkv.dtype)
    if storage is not None and storage.dtype != qkv.dtype:
      raise KernelError("cache and activations must share one dtype")
    self._call("sb_qk_norm_rotate_store", _ptr(qkv), qkv.shape[1], _code(qkv), _ptr(q_norm), _ptr(k_norm), float(eps),
               _ptr(head_scale), _ptr(rot_freq), 2 * rot_freq.numel() if rot_freq is not None else 0,
               _ptr(value_freq), _ptr(q), _ptr(storage), _ptr(block_table), block_table.shape[1],
               _ptr(ctx.token_seq), _ptr(ctx.positions), t, num_heads, num_kv_heads, head_dim, value_dim,
               ctx.page_size, storage.shape[0] if storage is not None else 0, int(storage is not None),
               _ptr(self.err))
    return q

  def pool_blocks(self, storage: torch.Tensor, block_table: torch.Tensor, pool_storage: torch.Tensor,
                  pool_table: torch.Tensor, ctx: Any, num_kv_heads: int, head_dim: int, value_dim: int,
                  pool: int) -> None:
    """Writes the mean key and value of every block of `pool` tokens that the step completes."""
    self._call("sb_pool_blocks", _ptr(storage), _code(storage), _ptr(block_table), block_table.shape[1],
               storage.shape[0], _ptr(pool_storage), _ptr(pool_table), pool_table.shape[1], pool_storage.shape[0],
               _ptr(ctx.cu_q), _ptr(ctx.q_start), ctx.num_seqs, ctx.max_q_len // pool + 1, num_kv_heads, head_dim,
               value_dim, ctx.page_size, pool, _ptr(self.err))

  def rotate_heads(self, x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, num_heads: int, dim: int,
                   inverse: bool = False) -> torch.Tensor:
    out = self._new(*x.shape, dtype=x.dtype)
    self._call("sb_rotate_heads", _ptr(x), _code(x), _ptr(positions), _ptr(freq), -1.0 if inverse else 1.0,
               x.shape[0], num_heads, dim, _ptr(out))
    return out

  # ---- attention with heads normed one by one ----------------------------------
  def rotate_headnorm_store(self, proj: torch.Tensor, eps: float, q_scale: float, rot_freq: torch.Tensor | None, *,
                            interleaved: bool, head_norm: bool, tie_values: bool, num_heads: int, num_kv_heads: int,
                            head_dim: int, storage: torch.Tensor | None, block_table: torch.Tensor,
                            ctx: Any, value_dim: int | None = None, bias: torch.Tensor | None = None) -> torch.Tensor:
    """proj [T, q | k | (v) | ...] -> queries [T, num_heads, head_dim], rotated, each head divided by
    its root mean square, times `q_scale`; keys (rotated, normed) and values (the keys as projected
    when `tie_values`, else the v columns) go into the pages of `storage` (csrc/attention_prepare.cu).
    `value_dim`: size of a value head where it is not the key heads'.  `bias`: float32 offsets of the
    q, k and v columns, added before the rotation."""
    t = proj.shape[0]
    value_dim = head_dim if value_dim is None else value_dim
    q = self._new(t, num_heads, head_dim, dtype=proj.dtype)
    if storage is not None and storage.dtype != proj.dtype:
      raise KernelError("cache and activations must share one dtype")
    self._call("sb_rotate_headnorm_store", _ptr(proj), proj.shape[1], _code(proj), _ptr(bias), float(eps), float(q_scale),
               _ptr(rot_freq), 2 * rot_freq.numel() if rot_freq is not None else 0, int(interleaved), int(head_norm),
               int(tie_values), _ptr(q), _ptr(storage), _ptr(block_table), block_table.shape[1],
               _ptr(ctx.token_seq), _ptr(ctx.positions), t, num_heads, num_kv_heads, head_dim, value_dim,
               ctx.page_size, storage.shape[0] if storage is not None else 0, int(storage is not None),
               _ptr(self.err))
    return q

  def sigmoid_gate(self, x: torch.Tensor, proj: torch.Tensor, offset: int, per: int = 1) -> torch.Tensor:
    """x [T, N] *= sigmoid(proj[:, offset : offset + N / per]), one gate per `per` neighbours, in place."""
    gate = proj[:, offset:]
    self._call("sb_sigmoid_gate", _ptr(x), gate.data_ptr(), proj.shape[1], _code(x), x.shape[0], x.shape[1], int(per))
    return x

  # ---- a residual stream kept several times -------------------------------------------------------
  def spread_streams(self, h: torch.Tensor, copies: int) -> torch.Tensor:
    lanes = self._new(h.shape[0], copies, h.shape[1], dtype=torch.float32)
    self._call("sb_spread_streams", _ptr(h), _ptr(lanes), h.shape[0], copies, h.shape[1])
    return lanes

  def streams_step(self, lanes: torch.Tensor, branch: torch.Tensor | None, mix, out_w, weights, norm_weight,
                   eps: float, plus_one: bool, rows: torch.Tensor | None) -> torch.Tensor | None:
    """lanes [T, S, W] float32.  With `branch`: lanes[:, t] <- sum_s mix[s, t] lanes[:, s] + out_w[t] branch
    (in place; with `rows` only those rows are computed and nothing is written).  With `weights`:
    returns rms(sum_s weights[s] lanes[:, s]) * norm_weight in the activation dtype (`norm_weight`
    None: the sum, float32).  One kernel (csrc/stream_mix.cu)."""
    t, copies, width = lanes.shape
    n = t if rows is None else rows.numel()
    if branch is not None and branch.dtype != self.dtype:
      branch = self.cast(branch, self.dtype)
    y = y_sum = None
    if weights is not None and norm_weight is not None:
      y = self._new(n, width)
    elif weights is not None:
      y_sum = self._new(n, width, dtype=torch.float32)
    self._call("sb_streams_step", _ptr(lanes), _ptr(branch), 0 if self.dtype == torch.float32 else 1, _ptr(mix),
               _ptr(out_w), _ptr(weights), _ptr(norm_weight),
               int(norm_weight is not None and norm_weight.dtype == torch.float32), float(eps), int(plus_one),
               _ptr(rows), n, _ptr(y), _ptr(y_sum), copies, width, t, _ptr(self.err))
    return y if y is not None else y_sum

  def short_conv(self, x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, state: torch.Tensor | None,
                 ctx: Any, *, activation: int = 0, residual: bool = False, offset: int = 0,
                 channels: int | None = None, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """Causal convolution over time per channel on x[:, offset : offset + channels] with the request's
    last taps - 1 inputs in `state` [slots, taps - 1, channels] (csrc/stream_mix.cu)."""
    channels = x.shape[1] - offset if channels is None else channels
    taps = weight.shape[1]
    out = self._new(x.shape[0], channels, dtype=out_dtype or self.dtype)
    if out.dtype not in (x.dtype, torch.float32):
      raise KernelError("a convolution's result is in its input's dtype or float32")
    self._call("sb_short_conv", _ptr(x), x.shape[1], offset, _code(x), _ptr(weight), _ptr(bias), _ptr(state),
               _ptr(ctx.token_seq), _ptr(ctx.cu_q), _ptr(ctx.slots), x.shape[0], ctx.num_seqs,
               state.shape[0] if state is not None else 0, taps, channels, int(activation), int(residual),
               int(out.dtype == torch.float32),
               _ptr(out), _ptr(self.err))
    self.launches += taps > 1
    return out

  def group_norm_gate(self, o: torch.Tensor, weight: torch.Tensor, eps: float, *, groups: int,
                      gate: torch.Tensor | None = None, gate_offset: int = 0, gate_kind: str = "none") -> torch.Tensor:
    """o float32 [T, N...], RMS-normed in `groups` equal parts, times weight [N]; the gate
    gate[:, gate_offset : gate_offset + N] acts as silu before the norm or as sigmoid after it."""
    t = o.shape[0]
    n = o.numel() // max(t, 1)
    kind = {"none": 0, "sigmoid_after": 1, "silu_before": 2}[gate_kind]
    if kind and gate.dtype != self.dtype:
      raise KernelError("the gate comes in the activation dtype")
    out = self._new(t, n)
    self._call("sb_group_norm_gate", _ptr(o), _ptr(gate) if kind else None, gate.shape[1] if kind else 0,
               gate_offset, kind, _code(out), _ptr(weight), float(eps), t, n, groups, _ptr(out))
    return out

  def tanh_columns(self, x: torch.Tensor, offset: int, n: int) -> torch.Tensor:
    out = self._new(x.shape[0], n, dtype=x.dtype)
    self._call("sb_tanh_columns", _ptr(x), x.shape[1], offset, n, _code(x), _ptr(out), x.shape[0])
    return out

  def head_linear(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [T, H * Din] . w [H, Dout, Din]^T per head -> [T, H * Dout] (csrc/stream_mix.cu)."""
    h, dout, din = w.shape
    if w.dtype != x.dtype:
      raise KernelError("a product per head takes weights in the activations' dtype")
    out = self._new(x.shape[0], h * dout, dtype=x.dtype)
    if not self._library_head_products(x, din, w, out, dout, 1.0):
      self._call("sb_head_linear", _ptr(x), h * din, din, 0, _ptr(w), _code(x), h, din, dout, _ptr(out), h * dout, dout,
                 1.0, x.shape[0])
    return out

  # ---- attention over latents ---------------------------------------------------------------------
  def latent_prepare(self, down: torch.Tensor, query_norm: torch.Tensor, kv_norm: torch.Tensor, eps: float,
                     freq: torch.Tensor | None, *, query_rank: int, kv_rank: int, rotated_dim: int,
                     storage: torch.Tensor | None, block_table: torch.Tensor, ctx: Any) -> torch.Tensor:
    """Norms of both latents, the shared key part turned, the token's row [c | k_r] into its page;
    returns the queries' latent [T, query_rank] (csrc/latent_attention.cu)."""
    t = down.shape[0]
    cq = self._new(t, query_rank, dtype=down.dtype)
    if storage is not None and storage.dtype != down.dtype:
      raise KernelError("the cache of latents is kept in the activation dtype")
    self._call("sb_latent_prepare", _ptr(down), down.shape[1], _code(down), _ptr(query_norm), _ptr(kv_norm),
               float(eps), _ptr(freq), freq.numel() if freq is not None else 0, query_rank, kv_rank, rotated_dim,
               _ptr(ctx.positions), _ptr(ctx.token_seq), _ptr(block_table), block_table.shape[1], ctx.page_size,
               storage.shape[0] if storage is not None else 0, _ptr(storage), _ptr(cq), t, _ptr(self.err))
    return cq

  def latent_queries(self, q: torch.Tensor, key_up_t: torch.Tensor, freq: torch.Tensor | None, scale: float,
                     ctx: Any, *, num_heads: int, head_dim: int, rotated_dim: int) -> torch.Tensor:
    """Per head [W_uk^T q_plain | turn(q_rot)] * scale: q [T, H (head_dim + rotated_dim)], key_up_t
    [H, kv_rank, head_dim] -> [T, H (kv_rank + rotated_dim)]."""
    t = q.shape[0]
    rank = key_up_t.shape[1]
    row_in, row_out = head_dim + rotated_dim, rank + rotated_dim
    out = self._new(t, num_heads * row_out, dtype=q.dtype)
    if not self._library_head_products(q, row_in, key_up_t, out, row_out, scale):
      self._call("sb_head_linear", _ptr(q), num_heads * row_in, row_in, 0, _ptr(key_up_t), _code(q), num_heads, head_dim,
                 rank, _ptr(out), num_heads * row_out, row_out, float(scale), t)
    self._call("sb_turn_query_part", _ptr(q), row_in, head_dim, _ptr(out), row_out, rank, _code(q), _ptr(freq),
               freq.numel() if freq is not None else 0, rotated_dim, float(scale), _ptr(ctx.positions), t, num_heads)
    return out

  # ---- recurrent mixers with a matrix per head ------------------------------------------------------
  def general_delta_scan(self, pre: torch.Tensor, low: torch.Tensor, decay_bias: torch.Tensor,
                         removal_bias: torch.Tensor, state: torch.Tensor, ctx: Any, *, num_heads: int,
                         head_dim: int) -> torch.Tensor:
    """pre [T, r | k | v | gate | a | ...], low [T, heads * head_dim] -> float32 o [T, heads, head_dim];
    walks every sequence's tokens through its state [slots, heads, head_dim, head_dim] (csrc/state_scans.cu)."""
    t = pre.shape[0]
    out = self._new(t, num_heads, head_dim, dtype=torch.float32)
    scratch = self._new(t, num_heads * (6 * head_dim + 2), dtype=torch.float32)
    self._call("sb_general_delta_scan", _ptr(pre), pre.shape[1], _ptr(low), low.shape[1], _code(pre), _ptr(decay_bias),
               _ptr(removal_bias), _ptr(state), _ptr(ctx.cu_q), _ptr(ctx.slots), t, ctx.num_seqs, state.shape[0],
               num_heads, head_dim, ctx.max_q_len, _ptr(scratch), _ptr(out), _ptr(self.err))
    self.launches += 1
    return out

  def state_space_scan(self, xbc: torch.Tensor, pre: torch.Tensor, step_offset: int, step_bias: torch.Tensor,
                       neg_rate: torch.Tensor, skip: torch.Tensor, state: torch.Tensor, ctx: Any, *, num_heads: int,
                       value_dim: int, state_dim: int, num_groups: int) -> torch.Tensor:
    """xbc float32 [T, x | B | C] after convolution and silu, the steps' sizes from pre[:, step_offset:]
    -> float32 y [T, heads, value_dim]; state [slots, heads, state_dim, value_dim] (csrc/state_scans.cu)."""
    t = xbc.shape[0]
    out = self._new(t, num_heads, value_dim, dtype=torch.float32)
    scratch = self._new(t, num_heads * 2, dtype=torch.float32)
    self._call("sb_state_space_scan", _ptr(xbc), xbc.shape[1], _ptr(pre), pre.shape[1], _code(pre), step_offset,
               _ptr(step_bias), _ptr(neg_rate), _ptr(skip), _ptr(state), _ptr(ctx.cu_q), _ptr(ctx.slots), t,
               ctx.num_seqs, state.shape[0], num_heads, num_groups, state_dim, value_dim, ctx.max_q_len,
               _ptr(scratch), _ptr(out), _ptr(self.err))
    self.launches += 1
    return out

  # ---- forget-gate recurrence ---------------------------------------------------
  def forget_gate_scan(self, pre: torch.Tensor, bias: torch.Tensor, lower: torch.Tensor, state: torch.Tensor,
                       ctx: Any, *, num_heads: int, head_dim: int, value_dim: int) -> torch.Tensor:
    """pre [T, q | f | v] as projected -> float32 o [T, heads, value_dim]; walks every sequence's
    tokens through its state [slots, heads, head_dim, value_dim] (csrc/recurrent_mix.cu)."""
    t = pre.shape[0]
    out = self._new(t, num_heads, value_dim, dtype=torch.float32)
    scratch = self._new(t, num_heads * (2 * head_dim + value_dim), dtype=torch.float32)  # activations, gates, values
    self._call("sb_forget_scan", _ptr(pre), pre.shape[1], _code(pre), _ptr(bias), _ptr(lower), _ptr(state),
               _ptr(ctx.cu_q), _ptr(ctx.slots), t, ctx.num_seqs, state.shape[0], num_heads, head_dim, value_dim,
               ctx.max_q_len, _ptr(scratch), _ptr(out), _ptr(self.err))
    self.launches += 1
    return out

  # ---- routed experts -------------------------------------------------------------
  MOE_TILE_ROWS = 64  # rows of a tile of the experts' products (csrc/moe.cu)

  def route_tokens(self, x: torch.Tensor, router: torch.Tensor, correction: torch.Tensor | None,
                   shared_gate_w: torch.Tensor | None, *, top: int, scale: float, score: int = 0,
                   renormalize: bool = False, bias: torch.Tensor | None = None):
    """Per token the `top` chosen experts (int32 [T, top]), their weights (float32 [T, top]) and the
    shared expert's gate (float32 [T], or None)."""
    t, width = x.shape
    chosen = self._new(t, top, dtype=torch.int32)
    weight = self._new(t, top, dtype=torch.float32)
    gate = self._new(t, dtype=torch.float32) if shared_gate_w is not None else None
    self._call("sb_moe_route", _ptr(x), _code(x), t, width, _ptr(router), _ptr(correction), _ptr(shared_gate_w),
               _ptr(bias), router.shape[0], top, float(scale), int(score), int(renormalize), _ptr(chosen), _ptr(weight), _ptr(gate))
    return chosen, weight, gate

  def route_by_table(self, token_ids: torch.Tensor, table: torch.Tensor, num_experts: int):
    """chosen[t, j] = table[id_t, j] (int32 [T, top]) and the weights 1 / top (float32 [T, top])."""
    t, top = token_ids.numel(), table.shape[1]
    chosen = self._new(t, top, dtype=torch.int32)
    weight = self._new(t, top, dtype=torch.float32)
    self._call("sb_table_route", _ptr(token_ids), _ptr(table), table.shape[0], top, num_experts, _ptr(chosen),
               _ptr(weight), t, _ptr(self.err))
    return chosen, weight

  def _experts_one_by_one(self, x, sorted_pair, tiles, top, gate_up, down, activation, gated=True,
                          limit: float = 0.0) -> torch.Tensor:
    """The experts' products of a long prompt portion: the rows, sorted by expert, are gathered once,
    the host reads how many each expert got (the one wait of the step), and every expert's rows go
    through the engine's own products for a dense feed-forward (the tcgen05 kernel with the
    activation on its sums from 129 rows, the library's product for the way down), issued by one
    native call that puts every other expert on a second stream (csrc/moe.cu).  Experts without a
    gate: the library's product both ways, the activation in place between them.  Returns the rows
    of every pair in sorted order, as the grouped kernel does."""
    expert, row0, count = tiles.cpu().numpy()
    total = int(count[expert >= 0].sum())  # (identity experts' pairs have no row; the list's tail is unused)
    rows_of = torch.div(sorted_pair[:total], top, rounding_mode="floor")
    xs = self.gather_rows(x, rows_of)
    which = np.unique(expert[expert >= 0]).astype(np.int32)
    starts = np.array([row0[expert == e].min() for e in which], dtype=np.int32)
    counts = np.array([count[expert == e].sum() for e in which], dtype=np.int32)
    width, hidden = x.shape[1], down.shape[2]
    y = self._new(total, width, dtype=x.dtype)
    # Experts with enough rows for the tcgen05 product: all of them in one call of the library, so
    # that the host pays one call, not two per expert.  The others through the kernel table's methods.
    if not gated:
      big = np.ones(len(counts), dtype=bool)
    else:
      big = counts >= self.gated_tc_min_rows if self.gated_tc_min_rows > 0 else np.zeros(len(counts), dtype=bool)
    rest = [(int(e), int(s), int(n)) for e, s, n in zip(which[~big], starts[~big], counts[~big])]
    which, starts, counts = (np.ascontiguousarray(a[big]) for a in (which, starts, counts))
    if len(which):
      stream = self._stream()
      workspace = self._library_workspaces.get(stream.value)
      if workspace is None:
        workspace = self._library_workspaces[stream.value] = torch.empty(32 << 20, dtype=torch.uint8, device=self.device)
      second = None
      if self.expert_side_stream:  # every other expert on a second stream, with a workspace of its own
        second = self._library_workspaces.get("experts")
        if second is None:
          second = self._library_workspaces["experts"] = torch.empty(32 << 20, dtype=torch.uint8, device=self.device)
      h = self._new(total, hidden, dtype=x.dtype)
      finished = ctypes.c_int(0)
      as_ints = lambda a: a.ctypes.data_as(ctypes.POINTER(ctypes.c_int))
      rc = self.lib.sb_experts_dense_bf16(
          _ptr(xs), _ptr(gate_up), _ptr(down), _ptr(h), _ptr(y), as_ints(starts), as_ints(counts), as_ints(which),
          len(which), width, hidden, activation, float(limit), int(gated), self.gated_tc_blocks, int(self.gated_tc_pairs), _ptr(workspace),
          _ptr(second), workspace.numel(), ctypes.byref(finished), _ptr(self.err), stream)
      if rc > 0:
        raise KernelError(f"sb_experts_dense_bf16: CUDA or cuBLAS status {rc}")
      done = finished.value
      if not gated and done < len(which):
        raise KernelError("sb_experts_dense_bf16: the library refused a product")
      self.launches += (2 if gated else 3) * done
      rest += list(zip(which[done:].tolist(), starts[done:].tolist(), counts[done:].tolist()))
    for e, start, n in rest:
      h_e = self.gated_linear(xs[start:start + n], gate_up[e], activation, limit)
      y[start:start + n] = self.linear(h_e, down[e])
    return y

  def mix_experts(self, x: torch.Tensor, chosen: torch.Tensor, weight: torch.Tensor, gate_up: torch.Tensor | None,
                  down: torch.Tensor | None, num_experts: int, activation: int, shared: torch.Tensor | None,
                  shared_gate: torch.Tensor | None, gated: bool = True, limit: float = 0.0) -> torch.Tensor:
    """sum_j weight[t, j] * expert(chosen[t, j])(x[t]) + shared_gate[t] * shared[t]; experts with an
    index >= num_experts return their input.  gate_up [E, 2F, W], down [E, W, F]; `gated` False:
    experts without a gate, W_down act(W_up x), with gate_up [E, F, W]."""
    t, width = x.shape
    top = chosen.shape[1]
    pairs = t * top
    out = self._new(t, width, dtype=x.dtype)
    pos = self._new(pairs, dtype=torch.int32)
    y_pair = None
    if num_experts > 0:
      if gate_up.dtype != x.dtype:
        raise KernelError("the experts' matrices and the activations must share one dtype")
      max_tiles = pairs // self.MOE_TILE_ROWS + min(num_experts, pairs)
      words = self._new(pairs + 3 * max_tiles, dtype=torch.int32)
      sorted_pair, tiles = words[:pairs], words[pairs:].view(3, max_tiles)
      self._call("sb_moe_group", _ptr(chosen), pairs, num_experts, max_tiles, _ptr(sorted_pair), _ptr(pos),
                 _ptr(tiles[0]), _ptr(tiles[1]), _ptr(tiles[2]))
      hidden = down.shape[2]
      # (whole 16-byte groups per row, so that an expert's slice of the rows starts on a boundary)
      if (x.dtype == torch.bfloat16 and 0 < self.expert_rows_for_dense_products * num_experts <= pairs
          and width % 8 == 0 and hidden % 8 == 0 and not torch.cuda.is_current_stream_capturing()):
        y_pair = self._experts_one_by_one(x, sorted_pair, tiles, top, gate_up, down, activation, gated, limit)
      else:
        h = self._new(pairs, hidden, dtype=x.dtype)
        self._call("sb_moe_product", _ptr(x), _ptr(sorted_pair), top, _ptr(gate_up), _code(x), int(gated), width, hidden,
                   _ptr(tiles[0]), _ptr(tiles[1]), _ptr(tiles[2]), max_tiles, activation, float(limit), _ptr(h))
        y_pair = self._new(pairs, width, dtype=x.dtype)
        self._call("sb_moe_product", _ptr(h), None, 1, _ptr(down), _code(x), 0, hidden, width,
                   _ptr(tiles[0]), _ptr(tiles[1]), _ptr(tiles[2]), max_tiles, -1, 0.0, _ptr(y_pair))
    else:
      pos.fill_(-1)
    if shared is not None and shared.dtype != x.dtype:
      shared = self.cast(shared, x.dtype)
    self._call("sb_moe_combine", _ptr(x), _ptr(y_pair), _code(x), _ptr(chosen), _ptr(weight), _ptr(pos), _ptr(shared),
               _ptr(shared_gate), num_experts, top, t, width, _ptr(out))
    return out

  # ---- gated delta rule -------------------------------------------------------
  def delta_rule_inputs(self, pre: torch.Tensor, low: torch.Tensor, conv_weight: torch.Tensor,
                        conv_state: torch.Tensor, decay_bias: torch.Tensor, neg_rate: torch.Tensor, ctx: Any, *,
                        conv_taps: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int):
    """Convolutions with their state, activations, unit vectors, decays and beta (csrc/recurrent_mix.cu):
    float32 q, k [T, kv heads, head_dim], v [T, heads, value_dim], decay [T, heads, head_dim], beta [T, heads]."""
    t = pre.shape[0]
    f32 = torch.float32
    q = self._new(t, num_kv_heads, head_dim, dtype=f32)
    k = self._new(t, num_kv_heads, head_dim, dtype=f32)
    v = self._new(t, num_heads, value_dim, dtype=f32)
    decay = self._new(t, num_heads, head_dim, dtype=f32)
    beta = self._new(t, num_heads, dtype=f32)
    self._call("sb_delta_inputs", _ptr(pre), pre.shape[1], _ptr(low), low.shape[1], _code(pre), _ptr(conv_weight),
               _ptr(conv_state), _ptr(decay_bias), _ptr(neg_rate), _ptr(ctx.token_seq), _ptr(ctx.cu_q),
               _ptr(ctx.slots), t, ctx.num_seqs, conv_state.shape[0], conv_taps, num_kv_heads, num_heads, head_dim,
               value_dim, _ptr(q), _ptr(k), _ptr(v), _ptr(decay), _ptr(beta), _ptr(self.err))
    self.launches += conv_taps > 1
    return q, k, v, decay, beta

  def gated_delta_scan(self, q, k, v, decay, beta, state: torch.Tensor, ctx: Any, *, num_heads: int,
                       num_kv_heads: int, head_dim: int, value_dim: int) -> torch.Tensor:
    """Walks every sequence's tokens through its state [slots, heads, head_dim, value_dim]; float32 o."""
    out = self._new(q.shape[0], num_heads, value_dim, dtype=torch.float32)
    self._call("sb_delta_scan", _ptr(q), _ptr(k), _ptr(v), _ptr(decay), _ptr(beta), _ptr(state), _ptr(ctx.cu_q),
               _ptr(ctx.slots), ctx.num_seqs, state.shape[0], num_kv_heads, num_heads, head_dim, value_dim,
               ctx.max_q_len, _ptr(out), _ptr(self.err))
    return out

  def gated_head_norm(self, o: torch.Tensor, low: torch.Tensor | None, gate_offset: int, weight: torch.Tensor,
                      eps: float, num_heads: int, value_dim: int) -> torch.Tensor:
    """Per head o / rms(o) * weight, times sigmoid(low[:, gate_offset + ...]); `low` None: no gate."""
    if low is None:
      out = self._new(o.shape[0], num_heads * value_dim)
      self._call("sb_gated_head_norm", _ptr(o), None, 0, -1, _code(out), _ptr(weight),
                 float(eps), o.shape[0], num_heads, value_dim, _ptr(out))
      return out
    out = self._new(o.shape[0], num_heads * value_dim, dtype=low.dtype)
    self._call("sb_gated_head_norm", _ptr(o), _ptr(low), low.shape[1], gate_offset, _code(low), _ptr(weight),
               float(eps), o.shape[0], num_heads, value_dim, _ptr(out))
    return out

  def normed_mean(self, branches: Sequence[torch.Tensor], scales: Sequence[torch.Tensor], eps: float) -> torch.Tensor:
    x = [b if b.dtype == self.dtype else self.cast(b, self.dtype) for b in branches]
    out = self._new(*x[0].shape)
    pad = [None] * (4 - len(x))
    self._call("sb_normed_mean", *[_ptr(b) for b in x], *pad, *[_ptr(w) for w in scales], *pad, len(x),
               _code(out), float(eps), x[0].shape[0], x[0].shape[1], _ptr(out))
    return out

  # ---- sampling -------------------------------------------------------------
  def sample(self, logits: torch.Tensor, temperature, top_k, top_p, seed, position, logprobs: bool = False):
    """One token per row of float32 logits; the other arguments are host sequences.  With
    `logprobs` also the float32 log-probability of each token under the distribution it was
    drawn from (0 for greedy rows): (tokens, logprobs)."""
    params = self.pack_sample_params(temperature, top_k, top_p, seed, position)
    dev_params = torch.from_numpy(params).to(self.device, non_blocking=True)
    if not logprobs:
      return self.sample_device(logits, dev_params)
    lp = self._new(logits.shape[0], dtype=torch.float32)
    return self.sample_device(logits, dev_params, logprobs_out=lp), lp

  @staticmethod
  def pack_sample_params(temperature, top_k, top_p, seed, position) -> np.ndarray:
    """The [R, 6] int32 words the sampling kernel reads (see csrc/sampling.cu)."""
    r = len(temperature)
    params = np.zeros((r, 6), dtype=np.int32)
    params[:, 0] = np.asarray(temperature, dtype=np.float32).view(np.int32)
    params[:, 1] = np.asarray(top_k, dtype=np.int32)
    params[:, 2] = np.asarray(top_p, dtype=np.float32).view(np.int32)
    seeds = np.asarray([int(s) & 0xFFFFFFFFFFFFFFFF for s in seed], dtype=np.uint64)
    params[:, 3] = (seeds & np.uint64(0xFFFFFFFF)).astype(np.uint32).view(np.int32)
    params[:, 4] = (seeds >> np.uint64(32)).astype(np.uint32).view(np.int32)
    params[:, 5] = np.asarray(position, dtype=np.int32)
    return params

  def sample_device(self, logits: torch.Tensor, dev_params: torch.Tensor, out: torch.Tensor | None = None,
                    logprobs_out: torch.Tensor | None = None, step_counter: torch.Tensor | None = None) -> torch.Tensor:
    """Sampling with the parameter words already on the device.  `logprobs_out` (float32 [R], or
    [steps, R] indexed by the device-side `step_counter`) receives the tokens' log-probabilities."""
    r, vocab = logits.shape
    if out is None:
      out = self._new(r, dtype=torch.int32)
    slices = self.lib.sb_sample_slices(r, vocab)
    scratch = self._new(r * (2 + 2 * slices), dtype=torch.int32)
    logits = logits.contiguous()
    self._call("sb_sample", _ptr(logits), _ptr(dev_params), _ptr(out), r, vocab, _ptr(scratch))
    self.launches += 2
    if logprobs_out is not None:
      self._call("sb_sample_logprobs", _ptr(logits), _ptr(dev_params), _ptr(out), _ptr(logprobs_out),
                 _ptr(step_counter), r, vocab, _ptr(scratch))
    return out

  def token_logprobs(self, logits: torch.Tensor, tokens: torch.Tensor, temperature: float, top_k: int,
                     top_p: float) -> torch.Tensor:
    """float32 [R]: the log-likelihood of tokens[r] under row r of `logits` with the sampling masks
    applied (simply/utils/sampling_lib.py:540-601): a greedy setting scores the argmax 0 and every
    other token -inf; otherwise the log-softmax of logits / temperature over the kept entries."""
    r, vocab = logits.shape
    logits = logits.contiguous()
    params = self.pack_sample_params([temperature] * r, [top_k] * r, [top_p] * r, [0] * r, [0] * r)
    dev_params = torch.from_numpy(params).to(self.device, non_blocking=True)
    slices = self.lib.sb_sample_slices(r, vocab)
    scratch = self._new(r * (2 + 2 * slices), dtype=torch.int32)
    drawn = self._new(r, dtype=torch.int32)
    # (the draw is not used, except for greedy rows, where it is the argmax; the call leaves the
    # rows' keep-thresholds in `scratch`)
    self._call("sb_sample", _ptr(logits), _ptr(dev_params), _ptr(drawn), r, vocab, _ptr(scratch))
    out = self._new(r, dtype=torch.float32)
    tokens = tokens.to(device=self.device, dtype=torch.int32).contiguous()
    self._call("sb_sample_logprobs", _ptr(logits), _ptr(dev_params), _ptr(tokens), _ptr(out), None, r, vocab,
               _ptr(scratch))
    if temperature == 0 or top_k == 1:
      out = torch.where(tokens == drawn, out, torch.full_like(out, float("-inf")))
    else:
      out = torch.where(out <= -3.0e38, torch.full_like(out, float("-inf")), out)  # a token the masks drop
    return out

  def keep_logits(self, logits: torch.Tensor, history: torch.Tensor, step_counter: torch.Tensor) -> None:
    """history[step_counter] = logits, without the host knowing the step (tests of graph replays)."""
    self._call("sb_keep_logits", _ptr(logits), _ptr(history), _ptr(step_counter), logits.numel())

  def decode_advance(self, sampled, token_ids, positions, q_start, sample_params, history, step_counter) -> None:
    self._call("sb_decode_advance", _ptr(sampled), _ptr(token_ids), _ptr(positions), _ptr(q_start),
               _ptr(sample_params), _ptr(history), _ptr(step_counter), sampled.numel())
