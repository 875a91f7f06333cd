"""Python entry points of the CUDA kernels.

Each function takes torch tensors that live on the CUDA device, checks what the
kernel cannot check cheaply (dtype, contiguity, sizes), and launches on torch's
current stream.  Nothing here computes on the CPU or falls back to a library
implementation; a failed launch raises ``KernelError``.

Kernels record out-of-range token ids, cache slots and block-table entries in a
device error word instead of trapping; ``check_errors`` reads it (one
synchronising copy) and raises.
"""

from __future__ import annotations

import ctypes
import dataclasses
import functools
from ctypes import c_float, c_int, c_int64, c_void_p

import numpy as np
import torch

from .library import KernelBuildError, load_library, require_cuda

SS_F32, SS_BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return SS_F32
    if dtype == torch.bfloat16:
        return SS_BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {dtype}")


_OPS_SIGNATURES = {
    "ss_embedding": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    "ss_gather_tokens": [c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "ss_prepare_decode": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64,
                          c_void_p],
    "ss_add_rmsnorm": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                       c_float, c_int, c_void_p],
    "ss_rope_cache": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                      c_int, c_int, c_int64, c_int, c_int, c_void_p, c_void_p],
    "ss_swiglu": [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p],
    "ss_gemm_simt": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int64,
                     c_int64, c_int, c_int, c_void_p],
    "ss_argmax": [c_void_p, c_void_p, c_int, c_int, c_int64, c_void_p, c_void_p, c_void_p],
    "ss_sample": [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "ss_mark_seen": [c_void_p, c_void_p, c_int, c_int, c_void_p],
    "ss_hc_norm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                   c_int, c_float, c_int, c_void_p, c_void_p],
    "ss_rope_norm_cache": [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_int,
                           c_int, c_int, c_int, c_float, c_int, c_int64, c_int, c_int, c_void_p, c_void_p],
    "ss_glu_limited": [c_void_p, c_void_p, c_int64, c_int, c_int, c_float, c_float, c_float, c_int, c_void_p],
    "ss_sigmoid_gate": [c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p],
    "ss_group_norm": [c_void_p, c_int, c_int64, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                      c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    "ss_round_stream": [c_void_p, c_void_p, c_int64, c_void_p],
    "ss_conv_silu": [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                     c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int],
    "ss_ssm_scan": [c_void_p, c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                    c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int],
    "ss_router": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p,
                  c_int, c_int, c_void_p, c_int],
    "ss_moe_plan": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int],
    "ss_moe_gemm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                    c_int, c_int, c_int, c_int, c_int, c_void_p, c_int],
    "ss_moe_gemm_mma": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                        c_int, c_int, c_int, c_int, c_void_p],
    "ss_moe_gather": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "ss_moe_combine": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
    "ss_norm_rope_cache": [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                           c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int64, c_int, c_void_p,
                           c_void_p],
    "ss_turn_heads": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "ss_soft_cap": [c_void_p, c_int64, c_float, c_void_p, c_float],
    "ss_embed_sum": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                     c_int, c_int, c_int, c_int, c_int, c_int64, c_int64, c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    "ss_matrix_cell": [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_float, c_float, c_void_p, c_void_p,
                       c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                       c_void_p, c_void_p],
    "ss_cell_output": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_float,
                       c_int, c_void_p],
    "ss_gated_recurrence": [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                            c_int, c_void_p, c_void_p, c_int],
    "ss_xielu": [c_void_p, c_void_p, c_int64, c_float, c_float, c_int, c_void_p],
    "ss_latent_rows": [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                       c_int, c_int, c_int, c_int, c_int, c_int, c_int64, c_float, c_int, c_void_p, c_void_p],
    "ss_decay_attention": [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                           c_int, c_int, c_int, c_void_p, c_void_p],
    "ss_gated_rmsnorm": [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p],
    "ss_block_gates": [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "ss_gated_linear_recurrence": [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_float, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int],
    "ss_head_gate": [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p],
    "ss_scaled_sum": [c_void_p, c_float, c_void_p, c_float, c_void_p, c_int64, c_int, c_void_p],
    "ss_relu_square": [c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_void_p],
    "ss_moe_mix": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_void_p,
                   c_int, c_int, c_int, c_int, c_void_p],
    "ss_head_product": [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_int,
                        c_int, c_void_p, c_void_p, c_float, c_void_p, c_int64, c_int, c_int, c_void_p],
}

_ATTN_SIGNATURES = {
    "ss_attn_simt": [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p,
                     c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_float,
                     c_int, c_int, c_void_p, c_void_p, c_void_p, c_float, c_void_p],
    "ss_attn_prefill_mma": [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p,
                            c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_float,
                            c_int, c_void_p, c_void_p, c_void_p, c_float, c_void_p],
    "ss_attn_prefill_tc5": [c_void_p, c_int64, c_int, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p,
                            c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_float, c_int, c_int,
                            c_void_p, c_void_p, c_float, c_void_p],
    "ss_attn_decode_tma": [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int,
                           c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_float, c_int, c_int,
                           c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_float],
    "ss_attn_decode_mma": [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int,
                           c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_float, c_int, c_int,
                           c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p],
}

_GEMM_SIGNATURES = {
    "ss_gemm_tc5_many": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64,
                         c_int, c_int, c_int, c_void_p, c_void_p],
    "ss_gemm_tc5_many_tile_cols": [c_int, c_int, c_int],
    "ss_gemm_tc5_many_to_stream": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int64, c_int,
                                   c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    "ss_gemm_tc5_many_scaled": [c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_void_p, c_int, c_int,
                                c_int, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_void_p, c_void_p],
    "ss_gemm_tc5": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64,
                    c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "ss_gemm_tc5_glu": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64,
                        c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_void_p, c_void_p, c_void_p, c_void_p],
    "ss_gemm_tc5_many_glu": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64,
                             c_float, c_float, c_float, c_void_p, c_void_p],
    "ss_gemm_tc5_to_stream": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int64, c_int, c_int,
                              c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    "ss_gemm_tc5_to_streams": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int64, c_int, c_int,
                               c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    "ss_gemm_tc5_scaled_glu": [c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                               c_int64, c_int64, c_int64, c_int, c_int, c_int, c_float, c_float, c_float, c_void_p, c_void_p,
                               c_void_p, c_void_p],
    "ss_gemm_tc5_grouped": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int64, c_int, c_void_p,
                            c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    "ss_gemm_tc5_scaled": [c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                           c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
}

_state: dict[str, object] = {}


def _declare(lib: ctypes.CDLL, table: dict[str, list]) -> None:
    for name, argtypes in table.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue
        fn.argtypes = argtypes
        fn.restype = c_int


def ops_library() -> ctypes.CDLL:
    lib = _state.get("ops")
    if lib is None:
        require_cuda()
        lib = load_library("slipstream_ops", ["ops.cu", "ops_streams.cu", "ops_mixers.cu", "ops_cells.cu", "ops_gated.cu", "sampling.cu"])
        _declare(lib, _OPS_SIGNATURES)
        _state["ops"] = lib
    return lib  # type: ignore[return-value]


def gemm_library() -> ctypes.CDLL:
    lib = _state.get("gemm")
    if lib is None:
        require_cuda()
        lib = load_library("slipstream_gemm", ["gemm_tc5.cu"])
        _declare(lib, _GEMM_SIGNATURES)
        _state["gemm"] = lib
    return lib  # type: ignore[return-value]


def attention_library(head_dim: int) -> ctypes.CDLL:
    key = f"attn{head_dim}"
    lib = _state.get(key)
    if lib is None:
        require_cuda()
        if head_dim % 16 != 0 or not (16 <= head_dim <= 256):
            raise KernelError(
                f"attention kernels take head sizes that are multiples of 16 up to 256, not {head_dim}")
        lib = load_library("slipstream_attn", ["attention.cu"], {"HEAD_DIM": head_dim})
        _declare(lib, _ATTN_SIGNATURES)
        _state[key] = lib
    return lib  # type: ignore[return-value]


def error_word(device: torch.device) -> torch.Tensor:
    key = ("err", device)
    word = _state.get(key)
    if word is None:
        with torch.inference_mode(False):  # the word is cleared in place later, from any mode
            word = torch.zeros(1, dtype=torch.int32, device=device)
        _state[key] = word
    return word  # type: ignore[return-value]


_ERR_NAMES = {1: "a token id outside the vocabulary", 2: "a cache slot outside the pool",
              4: "a block-table entry outside the pool", 8: "a bounded wait gave up"}


def raise_for_status(value: int, device: torch.device) -> None:
    """Raise ``KernelError`` for a non-zero value of the error word (already on the host) and clear the word."""
    if value:
        error_word(device).zero_()
        what = "; ".join(text for bit, text in _ERR_NAMES.items() if value & bit) or f"status {value}"
        raise KernelError(f"a kernel reported: {what}")


def check_errors(device: torch.device) -> None:
    raise_for_status(int(error_word(device).item()), device)


@functools.lru_cache(maxsize=None)
def _device_sm_count(index: int) -> int:
    return int(torch.cuda.get_device_properties(index).multi_processor_count)


def sm_count(device: torch.device | int | None = None) -> int:
    """Streaming multiprocessors of ``device`` (default: the current CUDA device), asked from the device once.
    Every rule below that sizes a grid or a split takes this number as ``sms``."""
    if isinstance(device, torch.device):
        device = device.index
    if device is None:
        require_cuda()
        device = torch.cuda.current_device()
    return _device_sm_count(int(device))


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """Handle of the current CUDA stream (every wrapper below asks for it, so the short way is taken when
    this torch has it)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


_launches = [0]


def launch_count() -> int:
    """Kernels of this package launched so far (each entry point below launches exactly one;
    a replayed CUDA graph adds the kernels it holds, see ``count_launches``)."""
    return _launches[0]


def count_launches(n: int) -> None:
    _launches[0] += n


def _check(code: int, what: str) -> None:
    _launches[0] += 1
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code} at launch")


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, dtype: torch.dtype | None, what: str) -> None:
    if not t.is_cuda:
        raise KernelError(f"{what} must be a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")


# --------------------------------------------------------------------------- model ops

def embedding(token_ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None, scale: float = 1.0,
              copies: int = 1) -> torch.Tensor:
    """Rows of ``table`` [vocab, hidden] at ``token_ids`` (int32 [N]), times ``scale``, as float32 [N, hidden]; with
    ``copies`` > 1 as [N, copies, hidden], every copy the same (the residual streams of a model that keeps several)."""
    _need(token_ids, torch.int32, "token_ids")
    _need(table, None, "embedding table")
    n, (vocab, hidden) = token_ids.numel(), table.shape
    shape = (n, hidden) if copies == 1 else (n, copies, hidden)
    if out is None:
        out = torch.empty(shape, dtype=torch.float32, device=table.device)
    _need(out, torch.float32, "embedding output")
    if out.numel() != n * copies * hidden:
        raise KernelError("embedding output has the wrong size")
    _check(ops_library().ss_embedding(token_ids.data_ptr(), table.data_ptr(), out.data_ptr(), n, hidden,
                                      vocab, _code(table.dtype), float(scale), int(copies),
                                      error_word(table.device).data_ptr(), _stream()), "embedding")
    return out


def gather_tokens(token_ids: torch.Tensor, src_rows: torch.Tensor, pending: torch.Tensor) -> None:
    """``token_ids[r] = pending[src_rows[r]]`` where ``src_rows[r] >= 0`` (int32 tensors on the device): token ids
    sampled by the step before that the host has not read yet."""
    for name, t in (("token_ids", token_ids), ("src_rows", src_rows), ("pending", pending)):
        _need(t, torch.int32, name)
    _check(ops_library().ss_gather_tokens(token_ids.data_ptr(), src_rows.data_ptr(), pending.data_ptr(),
                                          src_rows.numel(), _stream()), "gather_tokens")


def prepare_decode(token_ids: torch.Tensor, src_rows: torch.Tensor, pending: torch.Tensor | None,
                   tables: torch.Tensor, patch_idx: torch.Tensor, patch_val: torch.Tensor,
                   n_patches: torch.Tensor) -> None:
    """The launch in front of a replayed decode step: ``gather_tokens`` (when ``pending`` is given) and
    ``tables.view(-1)[patch_idx[i]] = patch_val[i]`` for ``i < n_patches[0]`` (all int32 tensors on the device;
    the number of patches is read on the device, so the launch is the same every step)."""
    for name, t in (("token_ids", token_ids), ("src_rows", src_rows), ("tables", tables), ("patch_idx", patch_idx),
                    ("patch_val", patch_val), ("n_patches", n_patches)):
        _need(t, torch.int32, name)
    if pending is not None:
        _need(pending, torch.int32, "pending")
    _check(ops_library().ss_prepare_decode(token_ids.data_ptr(), src_rows.data_ptr(), _ptr(pending),
                                           src_rows.numel(), tables.data_ptr(), patch_idx.data_ptr(),
                                           patch_val.data_ptr(), n_patches.data_ptr(), patch_idx.numel(),
                                           tables.numel(), _stream()), "prepare_decode")


def add_rmsnorm(residual: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: torch.Tensor | None = None,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """``residual`` (float32 [N, H]) += ``delta`` in place, then RMSNorm times ``weight``.

    With ``rows`` (int32 [M]) only those rows are produced and ``residual`` is not changed.
    ``weight`` is in ``out_dtype`` or float32."""
    _need(residual, torch.float32, "residual")
    hidden = residual.shape[-1]
    n_out = residual.shape[0] if rows is None else rows.numel()
    if delta is not None:
        _need(delta, out_dtype, "delta")
        if delta.shape != residual.shape:
            raise KernelError(f"delta {tuple(delta.shape)} does not match residual {tuple(residual.shape)}")
    _need(weight, None, "norm weight")
    if weight.numel() != hidden or weight.dtype not in (out_dtype, torch.float32):
        raise KernelError("norm weight has the wrong size or dtype")
    if rows is not None:
        _need(rows, torch.int32, "rows")
    if out is None:
        out = torch.empty((n_out, hidden), dtype=out_dtype, device=residual.device)
    _need(out, out_dtype, "norm output")
    w_f32 = int(weight.dtype == torch.float32 and out_dtype != torch.float32)
    _check(ops_library().ss_add_rmsnorm(residual.data_ptr(), _ptr(delta), weight.data_ptr(), w_f32,
                                        out.data_ptr(), _ptr(rows), n_out, hidden, float(eps),
                                        _code(out_dtype), _stream()), "add_rmsnorm")
    return out


def hc_norm(streams: torch.Tensor, y: torch.Tensor | None, mix: torch.Tensor | None, w_out: torch.Tensor | None,
            w_in: torch.Tensor | None, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows: torch.Tensor | None = None, y2: torch.Tensor | None = None) -> torch.Tensor:
    """One hyper-connection step on ``streams`` (float32 [N, S, H], changed in place).  Write: stream t becomes
    ``sum_s mix[s, t] * stream s + w_out[t] * y`` (skipped when ``y`` is None).  Read: ``u = sum_t w_in[t] * stream t``
    (``w_in`` None: the plain sum).  Norm: returns ``u / sqrt(mean(u^2) + eps) * weight`` in ``out_dtype`` [N, H],
    all in float32 with one rounding at the end.  ``mix`` [S, S], ``w_out`` [S], ``w_in`` [S]: float32 on the device.
    With ``rows`` (int32 [M]) only those tokens are produced and the streams are left as they are.  ``y2``: a second
    output of the same branch point (two branches that read one input); ``y + y2``, added in float32, is written."""
    _need(streams, torch.float32, "streams")
    if streams.dim() != 3:
        raise KernelError("streams must be [tokens, streams, hidden]")
    n, s, hidden = streams.shape
    if y is not None:
        _need(y, out_dtype, "branch output")
        if tuple(y.shape) != (n, hidden):
            raise KernelError(f"branch output {tuple(y.shape)} does not match the streams {tuple(streams.shape)}")
        _need(mix, torch.float32, "mix")
        _need(w_out, torch.float32, "w_out")
        if mix.numel() != s * s or w_out.numel() != s:
            raise KernelError("mix must be [S, S] and w_out [S]")
        if y2 is not None:
            _need(y2, out_dtype, "second branch output")
            if y2.shape != y.shape:
                raise KernelError("the two branch outputs differ in shape")
    elif y2 is not None:
        raise KernelError("a second branch output comes with a first")
    if w_in is not None:
        _need(w_in, torch.float32, "w_in")
        if w_in.numel() != s:
            raise KernelError("w_in must be [S]")
    _need(weight, None, "norm weight")
    if weight.numel() != hidden or weight.dtype not in (out_dtype, torch.float32):
        raise KernelError("norm weight has the wrong size or dtype")
    if rows is not None:
        _need(rows, torch.int32, "rows")
    n_out = n if rows is None else rows.numel()
    out = torch.empty((n_out, hidden), dtype=out_dtype, device=streams.device)
    w_f32 = int(weight.dtype == torch.float32 and out_dtype != torch.float32)
    _check(ops_library().ss_hc_norm(streams.data_ptr(), _ptr(y), _ptr(mix) if y is not None else None,
                                    _ptr(w_out) if y is not None else None, _ptr(w_in), weight.data_ptr(), w_f32,
                                    out.data_ptr(), _ptr(rows), n_out, s, hidden, float(eps), _code(out_dtype),
                                    _stream(), _ptr(y2)), "hc_norm")
    return out


def rope_norm_cache(rows: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor | None,
                    inv_freq: torch.Tensor | None, kv: torch.Tensor | None, n_q: int, n_kv: int, head_dim: int,
                    rotary_dim: int, *, interleaved: bool = False, mscale: float = 1.0, norm_dim: int = 0,
                    eps: float = 0.0, write_cache: bool = True) -> None:
    """Rotation, unit norm and page write for one layer's projected heads.  ``rows`` [N, width]: each row starts
    with ``n_q`` query heads, then ``n_kv`` key heads and ``n_kv`` value heads (``n_kv`` 0: queries only) of
    ``head_dim`` elements; whatever follows them in a row is left alone.  The first ``rotary_dim`` elements of
    queries and keys are rotated by position * ``inv_freq`` in pairs (2i, 2i+1) (``interleaved``) or
    (i, i + rotary_dim / 2), cosines and sines times ``mscale``; with ``norm_dim`` > 0 each query and key head is
    then divided by ``sqrt(sum(x^2) / norm_dim + eps)``.  Queries change in place; keys and values go to their
    pages ``kv`` [pages, 2, n_kv, page_size, head_dim] at ``slots`` (-1 or ``write_cache`` False: keys in place)."""
    _need(rows, None, "projected rows")
    _need(positions, torch.int32, "positions")
    n, width = rows.shape
    if width < (n_q + 2 * n_kv) * head_dim:
        raise KernelError("the projected rows are narrower than their heads")
    if head_dim % 2 or head_dim > 256 or rotary_dim % 2 or rotary_dim > head_dim:
        raise KernelError("head_dim must be even and at most 256, rotary_dim even and at most head_dim")
    if rotary_dim:
        _need(inv_freq, torch.float32, "inv_freq")
        if inv_freq.numel() != rotary_dim // 2:
            raise KernelError("inv_freq must hold rotary_dim / 2 values")
    write = bool(write_cache and n_kv and kv is not None and slots is not None)
    pages = page_size = 0
    if write:
        _need(kv, rows.dtype, "kv pages")
        _need(slots, torch.int32, "slots")
        if kv.dim() != 5 or kv.shape[1] != 2 or kv.shape[2] != n_kv or kv.shape[4] != head_dim:
            raise KernelError(f"kv pages have shape {tuple(kv.shape)}, expected [pages, 2, {n_kv}, page, {head_dim}]")
        pages, page_size = kv.shape[0], kv.shape[3]
    _check(ops_library().ss_rope_norm_cache(rows.data_ptr(), width, positions.data_ptr(), _ptr(slots) if write else None,
                                            _ptr(inv_freq) if rotary_dim else None, float(mscale),
                                            _ptr(kv) if write else None, n, n_q, n_kv, head_dim, rotary_dim,
                                            int(interleaved), int(norm_dim), float(eps), max(page_size, 1), pages,
                                            int(write), _code(rows.dtype), error_word(rows.device).data_ptr(),
                                            _stream()), "rope_norm_cache")


def glu_limited(gate_up: torch.Tensor, block: int | None = None, alpha: float = 1.0, limit: float = 0.0,
                shift: float = 0.0) -> torch.Tensor:
    """``g * sigmoid(alpha * g) * (u + shift)`` with ``g = min(gate, limit)`` and ``u = clamp(up, -limit, limit)``
    (``limit`` 0: unclamped) for ``gate_up`` [N, 2 * I] laid out as for `swiglu`."""
    _need(gate_up, None, "gate_up")
    n, two_i = gate_up.shape
    inter = two_i // 2
    block = inter if block is None else block
    if block < 1 or inter % block:
        raise KernelError(f"block {block} does not divide the {inter} features")
    out = torch.empty((n, inter), dtype=gate_up.dtype, device=gate_up.device)
    _check(ops_library().ss_glu_limited(gate_up.data_ptr(), out.data_ptr(), n, inter, block, float(alpha), float(limit),
                                        float(shift), _code(gate_up.dtype), _stream()), "glu_limited")
    return out


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor) -> None:
    """``x *= sigmoid(gate)`` element by element; both [N, width], rows of either may be strided views."""
    if x.dtype != gate.dtype or x.shape != gate.shape or x.dim() != 2 or x.stride(1) != 1 or gate.stride(1) != 1:
        raise KernelError("sigmoid_gate takes two [N, width] tensors of one dtype with unit inner stride")
    if not x.is_cuda:
        raise KernelError("sigmoid_gate takes CUDA tensors")
    _check(ops_library().ss_sigmoid_gate(x.data_ptr(), x.stride(0), gate.data_ptr(), gate.stride(0), x.shape[0],
                                         x.shape[1], _code(x.dtype), _stream()), "sigmoid_gate")


def key_span(window: int | None = 0, chunk: int | None = 0) -> int:
    """The one integer the attention kernels take for what a query sees besides the causal rule: ``window`` W > 0,
    the last W keys; ``chunk`` C > 0, the keys of the query's own chunk of C positions (counted from the request's
    first token), passed as -C; neither: 0, every earlier key."""
    window, chunk = int(window or 0), int(chunk or 0)
    if window < 0 or chunk < 0:
        raise KernelError("window and chunk must not be negative")
    if window and chunk:
        raise KernelError("the attention kernels take a window or a chunk, not both")
    return window if window else -chunk


def rope_and_cache(qkv: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor | None,
                   inv_freq: torch.Tensor | None, kv: torch.Tensor | None, n_q: int, n_kv: int,
                   head_dim: int, rotary_dim: int, write_cache: bool = True) -> None:
    """Rotate queries (in place) and keys of ``qkv`` [N, (n_q + 2 n_kv) * D] by their positions and
    write keys and values to their pages: ``kv`` is [pages, 2, n_kv, page_size, D], ``slots`` int32 [N]
    = page * page_size + offset (-1 skips a token).  ``rotary_dim`` 0 copies without rotating."""
    _need(qkv, None, "qkv")
    _need(positions, torch.int32, "positions")
    n = qkv.shape[0]
    if qkv.shape[1] != (n_q + 2 * n_kv) * head_dim:
        raise KernelError("qkv has the wrong width")
    if rotary_dim % 2 or rotary_dim > head_dim:
        raise KernelError("rotary_dim must be even and at most head_dim")
    if rotary_dim:
        _need(inv_freq, torch.float32, "inv_freq")
        if inv_freq.numel() != rotary_dim // 2:
            raise KernelError("inv_freq must hold rotary_dim / 2 values")
    write = bool(write_cache and kv is not None and slots is not None)
    pages = page_size = 0
    if write:
        _need(kv, qkv.dtype, "kv pages")
        _need(slots, torch.int32, "slots")
        if kv.dim() != 5 or kv.shape[1] != 2 or kv.shape[2] != n_kv or kv.shape[4] != head_dim:
            raise KernelError(f"kv pages have shape {tuple(kv.shape)}, expected [pages, 2, {n_kv}, page, {head_dim}]")
        pages, page_size = kv.shape[0], kv.shape[3]
    _check(ops_library().ss_rope_cache(qkv.data_ptr(), positions.data_ptr(), _ptr(slots) if write else None,
                                       _ptr(inv_freq), _ptr(kv) if write else None, n, n_q, n_kv, head_dim,
                                       rotary_dim, max(page_size, 1), pages, int(write), _code(qkv.dtype),
                                       error_word(qkv.device).data_ptr(), _stream()), "rope_and_cache")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor | None = None, block: int | None = None) -> torch.Tensor:
    """``silu(gate) * up`` for ``gate_up`` = [N, 2 * I].  Gate and up features alternate in runs of ``block``
    columns (gate run, up run, gate run, ...); the default, ``block`` = I, is the plain [gate | up]."""
    _need(gate_up, None, "gate_up")
    n, two_i = gate_up.shape
    inter = two_i // 2
    block = inter if block is None else block
    if block < 1 or inter % block:
        raise KernelError(f"block {block} does not divide the {inter} features")
    if out is None:
        out = torch.empty((n, inter), dtype=gate_up.dtype, device=gate_up.device)
    _need(out, gate_up.dtype, "swiglu output")
    _check(ops_library().ss_swiglu(gate_up.data_ptr(), out.data_ptr(), n, inter, block, _code(gate_up.dtype),
                                   _stream()), "swiglu")
    return out


def gemm_simt(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
              out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ weight.T + bias`` on CUDA cores with float32 accumulation (no tensor cores):
    x [M, K], weight [N, K].  The float32 path of every projection."""
    _need(x, None, "x")
    _need(weight, x.dtype, "weight")
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"weight {tuple(weight.shape)} does not match x {tuple(x.shape)}")
    out_dtype = out_dtype or x.dtype
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    _need(out, out_dtype, "gemm output")
    bias_f32 = 0
    if bias is not None:
        _need(bias, None, "bias")
        bias_f32 = int(bias.dtype == torch.float32)
        if bias.numel() != n or (not bias_f32 and bias.dtype != x.dtype):
            raise KernelError("bias has the wrong size or dtype")
    _check(ops_library().ss_gemm_simt(x.data_ptr(), weight.data_ptr(), _ptr(bias), bias_f32, out.data_ptr(),
                                      m, n, k, k, n, _code(x.dtype), _code(out_dtype), _stream()), "gemm_simt")
    return out


def _check_sinks(sinks: torch.Tensor | None, n_q: int) -> None:
    if sinks is not None:
        _need(sinks, torch.float32, "sinks")
        if sinks.numel() != n_q:
            raise KernelError("sinks must hold one value per query head")


def _gate_ptr(gate: torch.Tensor | None, q: torch.Tensor, q_stride: int) -> int | None:
    if gate is None:
        return None
    if gate.dtype != q.dtype or gate.dim() != 2 or gate.stride(1) != 1 or gate.stride(0) != q_stride or not gate.is_cuda:
        raise KernelError("the gate must be a view of the projected rows: same dtype, unit inner stride, rows q_stride apart")
    return gate.data_ptr()


def paged_attention_simt(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv: torch.Tensor,
                         block_tables: torch.Tensor, tile_req: torch.Tensor, tile_q0: torch.Tensor,
                         q_start: torch.Tensor, seq_lens: torch.Tensor, n_q: int, n_kv: int,
                         head_dim: int, scale: float, window: int = 0, chunk: int = 0,
                         gate: torch.Tensor | None = None, softcap: float = 0.0,
                         sinks: torch.Tensor | None = None) -> None:
    """Causal grouped-query attention of the step's query rows over the pages (``window`` / ``chunk``: `key_span`).
    ``softcap`` c > 0 (in every attention entry point but the tcgen05 one): a scaled score s enters the softmax as
    ``c * tanh(s / c)``.
    ``gate`` (in every attention entry point): a view of the same rows as ``q`` ([N, n_q * D], rows ``q_stride``
    apart); the output is multiplied by its sigmoid as it is written.

    ``q`` points at the first query head of row 0; rows are ``q_stride`` elements apart.
    ``out`` is [N, n_q * D].  ``tile_req`` / ``tile_q0`` list tiles of 16 consecutive query tokens
    of one request (request index, first token within the request's rows of this step).
    ``sinks`` (in this entry point and the two mma.sync ones; float32 [n_q]): the softmax's denominator of head h also
    holds ``exp(sinks[h])``, a term of its own with neither key nor value, which the scale does not touch."""
    _need(out, q.dtype, "attention output")
    _check_sinks(sinks, n_q)
    _need(kv, q.dtype, "kv pages")
    for name, t in (("block_tables", block_tables), ("tile_req", tile_req), ("tile_q0", tile_q0),
                    ("q_start", q_start), ("seq_lens", seq_lens)):
        _need(t, torch.int32, name)
    lib = attention_library(head_dim)
    _check(lib.ss_attn_simt(q.data_ptr(), q_stride, out.data_ptr(), out.shape[1], kv.data_ptr(),
                            block_tables.data_ptr(), block_tables.shape[1], tile_req.data_ptr(),
                            tile_q0.data_ptr(), tile_req.numel(), q_start.data_ptr(), seq_lens.data_ptr(),
                            n_q, n_kv, kv.shape[3], kv.shape[0], float(scale), key_span(window, chunk),
                            _code(q.dtype), _gate_ptr(gate, q, q_stride), error_word(q.device).data_ptr(), _stream(),
                            float(softcap or 0.0), _ptr(sinks)),
           "paged_attention_simt")


def paged_attention_prefill(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv: torch.Tensor,
                            block_tables: torch.Tensor, tile_req: torch.Tensor, tile_row0: torch.Tensor,
                            q_start: torch.Tensor, seq_lens: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                            scale: float, window: int = 0, chunk: int = 0, gate: torch.Tensor | None = None,
                            softcap: float = 0.0, sinks: torch.Tensor | None = None) -> None:
    """bfloat16 tensor-core attention for prompt portions and mixed batches.  A tile is 64 consecutive
    rows of one request, a row being a (query token, head of the kv group) pair in token-major order:
    ``tile_req`` / ``tile_row0`` list (request index, first row)."""
    _need(out, torch.bfloat16, "attention output")
    _need(kv, torch.bfloat16, "kv pages")
    _check_sinks(sinks, n_q)
    if q.dtype != torch.bfloat16:
        raise KernelError("the tensor-core attention kernels take bfloat16")
    for name, t in (("block_tables", block_tables), ("tile_req", tile_req), ("tile_row0", tile_row0),
                    ("q_start", q_start), ("seq_lens", seq_lens)):
        _need(t, torch.int32, name)
    lib = attention_library(head_dim)
    _check(lib.ss_attn_prefill_mma(q.data_ptr(), q_stride, out.data_ptr(), out.shape[1], kv.data_ptr(),
                                   block_tables.data_ptr(), block_tables.shape[1], tile_req.data_ptr(),
                                   tile_row0.data_ptr(), tile_req.numel(), q_start.data_ptr(), seq_lens.data_ptr(),
                                   n_q, n_kv, kv.shape[3], kv.shape[0], float(scale), key_span(window, chunk),
                                   _gate_ptr(gate, q, q_stride), error_word(q.device).data_ptr(), _stream(),
                                   float(softcap or 0.0), _ptr(sinks)),
           "paged_attention_prefill")


def tcgen05_attention_fits(head_dim: int, n_q: int, n_kv: int, page_size: int, window: int) -> bool:
    """Whether the TMA-fed decode attention kernel takes this layer (``window`` 0), or the tcgen05 prefill kernel
    without a sliding window: head size 64 or 128, pages of 8, 16, 32 or 64 tokens, at most 128 query heads per kv
    head.  (The prefill kernel also takes windows, chunked masks and soft caps: `tcgen05_prefill_fits`.)"""
    return (head_dim in (64, 128) and not window and page_size in (8, 16, 32, 64) and n_q // n_kv <= 128)


def tcgen05_prefill_fits(head_dim: int, n_q: int, n_kv: int, page_size: int) -> bool:
    """Whether the tcgen05 prefill attention kernel takes this layer, whatever its mask (a sliding window, a chunked
    mask or none: the kernel starts at the first key tile a query tile can see and masks by row) and with or without
    a soft cap on the scores."""
    return tcgen05_attention_fits(head_dim, n_q, n_kv, page_size, 0)


def paged_attention_prefill_tcgen05(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv: torch.Tensor,
                                    block_tables: torch.Tensor, tile_req: torch.Tensor, tile_tok0: torch.Tensor,
                                    q_start: torch.Tensor, seq_lens: torch.Tensor, n_q: int, n_kv: int,
                                    head_dim: int, scale: float, key_parts: int = 1, chunk: int = 0, window: int = 0,
                                    softcap: float = 0.0, sinks: torch.Tensor | None = None) -> None:
    """bfloat16 causal attention for prompt portions and mixed batches on the tcgen05 tensor cores (Q, K, V
    tiles by TMA, S and O in tensor memory).  A tile is ``128 // (n_q // n_kv)`` consecutive query tokens of
    one request: ``tile_req`` / ``tile_tok0`` list (request index, first token within the request's rows); blocks
    start in list order, so the list should begin with the tiles that see the most keys.
    ``key_parts`` (1, 2, 4 or 8): the keys of every query tile are shared by that many blocks, a thread-block
    cluster whose results are combined through shared memory (see ``prefill_key_parts``).  ``chunk`` C: a query sees
    only the earlier keys of its own chunk of C positions; the key tiles in front of a query tile's first chunk are
    never fetched.  ``sinks`` (float32 [n_q]): one more term ``exp(sinks[h])`` in the denominator of head h, added where
    a row's sum is complete (by the block that writes the row, or once where a cluster combines its parts)."""
    _need(out, torch.bfloat16, "attention output")
    _check_sinks(sinks, n_q)
    _need(kv, torch.bfloat16, "kv pages")
    if q.dtype != torch.bfloat16:
        raise KernelError("the tensor-core attention kernels take bfloat16")
    if not tcgen05_attention_fits(head_dim, n_q, n_kv, kv.shape[3], 0):
        raise KernelError("the tcgen05 attention kernel does not take this head size or page size")
    for name, t in (("block_tables", block_tables), ("tile_req", tile_req), ("tile_tok0", tile_tok0),
                    ("q_start", q_start), ("seq_lens", seq_lens)):
        _need(t, torch.int32, name)
    lib = attention_library(head_dim)
    _check(lib.ss_attn_prefill_tc5(q.data_ptr(), q_stride, q.shape[0], out.data_ptr(), out.shape[1], kv.data_ptr(),
                                   block_tables.data_ptr(), block_tables.shape[1], tile_req.data_ptr(),
                                   tile_tok0.data_ptr(), tile_req.numel(), q_start.data_ptr(), seq_lens.data_ptr(),
                                   n_q, n_kv, kv.shape[3], kv.shape[0], float(scale), int(key_parts),
                                   key_span(window, chunk), error_word(q.device).data_ptr(), _stream(),
                                   float(softcap or 0.0), _ptr(sinks)),
           "paged_attention_prefill_tcgen05")


def prefill_key_parts(q_lens: np.ndarray, seq_lens: np.ndarray, tile_tokens: int, n_kv: int,
                      sms: int | None = None, span: int = 0) -> int:
    """Into how many parts the tcgen05 prefill kernel should cut the keys of its query tiles.  A block walks its
    key tiles one after the other, about a microsecond each, so a step with few query tiles lasts as long as its
    longest one while most SMs idle: a portion of 64 tokens behind 4,096 cached ones is 16 blocks of 64 key
    tiles, 47.5 us; with the keys of every query tile shared by 8 blocks 19.3 us; 512 tokens behind 4,096: 52.3
    against 41.5 us with 2.  Parts are only worth it while all blocks still run at once (every block pays for
    its own set-up and for the combination: a whole prompt of 2,048 tokens, 456 blocks, takes 47.5 us in one
    part and 59.3 in two) and while a part keeps 8 key tiles."""
    q_lens = np.asarray(q_lens, dtype=np.int64)
    seq_lens = np.asarray(seq_lens, dtype=np.int64)
    if q_lens.size == 0:
        return 1
    counts = (q_lens + tile_tokens - 1) // tile_tokens
    blocks = int(counts.sum()) * n_kv
    longest = int(seq_lens.max() - 1) // 64 + 1  # key tiles of the last query tile of the longest request
    if span > 0:  # under a window or a chunked mask a query tile sees no more than this many
        longest = min(longest, (span + tile_tokens) // 64 + 2)
    sms = sms or sm_count()
    parts = 1
    while parts < 8 and blocks * parts * 2 <= 2 * sms and longest >= 16 * parts:
        parts *= 2
    return parts


_DECODE_COUNTERS = 65536


def decode_counters(device: torch.device) -> torch.Tensor:
    """Counters of the split decode kernel (one per request and head block): zero between launches, which
    the kernel itself restores, so one tensor per device serves every call."""
    key = f"decode_counters{device}"
    counters = _state.get(key)
    if counters is None:
        counters = torch.zeros(_DECODE_COUNTERS, dtype=torch.int32, device=device)
        _state[key] = counters
    return counters  # type: ignore[return-value]


def decode_scratch(n_requests: int, n_q: int, n_slices: int, head_dim: int, device: torch.device):
    """Scratch memory of the split decode kernel: partial outputs and their log-sum-exps."""
    return (torch.empty((n_requests, n_q, n_slices, head_dim), dtype=torch.float32, device=device),
            torch.empty((n_requests, n_q, n_slices), dtype=torch.float32, device=device))


def paged_attention_decode(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv: torch.Tensor,
                           block_tables: torch.Tensor, q_start: torch.Tensor, seq_lens: torch.Tensor,
                           n_requests: int, n_q: int, n_kv: int, head_dim: int, scale: float, window: int = 0,
                           n_slices: int = 1, scratch: tuple[torch.Tensor, torch.Tensor] | None = None,
                           rope: tuple[torch.Tensor | None, int] | None = None, tma: bool | None = None,
                           stages: int = 2, chunk: int = 0, gate: torch.Tensor | None = None,
                           softcap: float = 0.0, sinks: torch.Tensor | None = None) -> None:
    """bfloat16 attention for requests that bring ONE token each, the keys of every request cut into
    ``n_slices`` slices that run in parallel.  Up to 8 slices form a thread-block cluster and are combined
    through shared memory; with more, the partial results (of every cluster of 8 in the TMA-fed kernel when the
    count is a multiple of 8, else of every slice) pass through ``scratch`` (see ``decode_scratch``) and the
    block that finishes a head block last combines them.

    ``rope`` = (inverse frequencies, rotary_dim): ``q`` is then the stacked projection output
    [N, (n_q + 2 n_kv) * D] as projected, and the kernel itself rotates queries and the newest key by each
    request's last position and writes the newest key and value to their page (what ``rope_and_cache`` does
    for other steps).

    ``tma``: the kernel whose tiles are moved by TMA (head size 64 or 128, pages of 8, 16, 32 or 64 tokens;
    the default where it fits), or the one that moves them with cp.async (every head and page size).
    ``stages``: 2 or 3 tiles in the ring of the TMA-fed kernel."""
    fits = tcgen05_attention_fits(head_dim, n_q, n_kv, kv.shape[3], 0) and sinks is None
    _check_sinks(sinks, n_q)
    if tma is None:
        tma = fits
    elif tma and not fits:
        raise KernelError("the TMA decode kernel takes head size 64 or 128 and pages of 8, 16, 32 or 64 tokens")
    _need(out, torch.bfloat16, "attention output")
    _need(kv, torch.bfloat16, "kv pages")
    if q.dtype != torch.bfloat16:
        raise KernelError("the tensor-core attention kernels take bfloat16")
    for name, t in (("block_tables", block_tables), ("q_start", q_start), ("seq_lens", seq_lens)):
        _need(t, torch.int32, name)
    part_o = part_lse = counters = None
    if n_slices > 8:
        counters = decode_counters(q.device)
        if n_requests * n_kv * ((n_q // n_kv + 15) // 16) > _DECODE_COUNTERS:
            raise KernelError("too many (request, head block) pairs for the decode counters")
        if scratch is None:
            scratch = decode_scratch(n_requests, n_q, n_slices, head_dim, q.device)
        part_o, part_lse = scratch
        if part_o.numel() < n_requests * n_q * n_slices * head_dim or part_lse.numel() < n_requests * n_q * n_slices:
            raise KernelError("decode scratch is too small")
    inv_freq, rotary_dim = rope if rope is not None else (None, 0)
    if rope is not None:
        if q_stride != (n_q + 2 * n_kv) * head_dim:
            raise KernelError("the fused rotation takes the stacked q/k/v projection")
        if rotary_dim % 2 or rotary_dim > head_dim:
            raise KernelError("rotary_dim must be even and at most head_dim")
        if rotary_dim:
            _need(inv_freq, torch.float32, "inv_freq")
            if inv_freq.numel() != rotary_dim // 2:
                raise KernelError("inv_freq must hold rotary_dim / 2 values")
    lib = attention_library(head_dim)
    args = (q.data_ptr(), q_stride, out.data_ptr(), out.shape[1], kv.data_ptr(), block_tables.data_ptr(),
            block_tables.shape[1], n_requests, q_start.data_ptr(), seq_lens.data_ptr(), n_q, n_kv, kv.shape[3], kv.shape[0],
            float(scale), key_span(window, chunk), n_slices, _ptr(inv_freq) if rotary_dim else None, rotary_dim,
            int(rope is not None), _ptr(part_o), _ptr(part_lse), _ptr(counters))
    if gate is not None and rope is not None:
        raise KernelError("a gated layer does not rotate inside the decode kernel")
    tail = (_gate_ptr(gate, q, q_stride), error_word(q.device).data_ptr(), _stream(), float(softcap or 0.0))
    if tma:
        _check(lib.ss_attn_decode_tma(*args, int(stages), *tail), "paged_attention_decode")
    else:
        _check(lib.ss_attn_decode_mma(*args, *tail, _ptr(sinks)), "paged_attention_decode")


WIDE_CONTEXT = 8192  # from this many cached tokens a decode step of few requests may use more than 8 slices


def is_long_context(seq_len: int) -> bool:
    return seq_len >= WIDE_CONTEXT


def decode_slices(n_requests: int, n_kv: int, group: int, max_seq_len: int, wide: bool = False,
                  sms: int | None = None) -> int:
    """How many slices to cut the keys into: as many as keep all blocks resident at once (two per SM),
    so that the step is one wave of blocks; at most 8, the size of a thread-block cluster.

    ``wide`` (the TMA-fed kernel, long contexts): few requests leave most SMs idle with 8 slices (one request on
    4 kv heads: 32 blocks), so the slices become 2, 4 or 8 clusters of 8 whose results meet in scratch memory,
    as long as a slice keeps 8 tiles of 64 keys and all blocks still fit one wave.  One request of 32,768 tokens:
    64.7 us with 8 slices, 23.4 us with 64; two of 16,384: 35.8 against 27.7 with 32; with 32 blocks or more
    (8 requests) 8 slices are the fastest at every length."""
    sms = sms or sm_count()
    blocks = n_requests * n_kv * ((group + 15) // 16)
    tiles = max(1, (max_seq_len + 63) // 64)
    most = max(1, min((2 * sms) // blocks, tiles, 8))
    # a power of two: clusters of 3 blocks pack the SMs of a GPC badly (24 requests x 4 kv heads: 24.8 us with 3
    # slices, 17.2 us with 2)
    slices = 1 << (most.bit_length() - 1)
    if wide and slices == 8:
        clusters = max(1, min((2 * sms) // (blocks * 8), tiles // 64, 8))
        slices = 8 * (1 << (clusters.bit_length() - 1))
    return slices


# Tiles of keys and values in the ring of a block of the TMA-fed decode attention.  With two, each pair of warps has
# one buffer and cannot fetch its next tile before it is done with this one: a block that walks many tiles (64
# requests of 1,024 tokens: 16 each) moves a tile per pair in the time of its products plus a trip to memory.  With
# three the third fills while both pairs work: a decode step of 64 requests 3.68 -> 3.62 ms, of 64 at 4,000 tokens
# 5.51 -> 5.27, of 32 at 16,000 7.78 -> 7.31, of 8 at 30,000 4.85 -> 4.65, of 8 at 1,024 2.70 -> 2.69.
DECODE_RING_STAGES = 3


def fuses_rope(qkv: torch.Tensor, ctx, head_dim: int, n_q: int, n_kv: int, page_size: int) -> bool:
    """Whether ``paged_attention`` should do the rotation and the page write of this step itself (``rope=``):
    bfloat16 steps in which every request brings one token.  With the TMA-fed decode kernel always (3.90
    against 3.94 ms a step at 64 requests, 3.01 against 3.08 at 8); with the cp.async one only up to the batch
    at which the projection before it is the tcgen05 kernel, since behind the library product the separate
    rotary kernel is what lets the attention kernel fetch cached keys early (4.18 against 4.28 ms at 64)."""
    if qkv.dtype != torch.bfloat16 or not ctx.is_decode_only:
        return False
    return tcgen05_attention_fits(head_dim, n_q, n_kv, page_size, 0) or qkv.shape[0] <= CLUSTER_BATCH


def paged_attention(qkv: torch.Tensor, out: torch.Tensor, kv: torch.Tensor, block_tables: torch.Tensor,
                    ctx, n_q: int, n_kv: int, head_dim: int, scale: float, window: int = 0,
                    rope: tuple[torch.Tensor | None, int] | None = None, chunk: int = 0,
                    gate: torch.Tensor | None = None, softcap: float = 0.0, sinks: torch.Tensor | None = None) -> None:
    """Attention of the step's rows over the pages, choosing the kernel for the batch.

    ``qkv`` is the stacked projection output [N, (n_q + 2 n_kv) * D] whose first n_q heads are the
    rotated queries; ``ctx`` gives the rows of each request (``q_start``), the cached lengths after
    this step (``seq_lens``) and the lists of query tiles.  float32 runs the CUDA-core kernel;
    bfloat16 the tensor-core kernels: the split decode kernel when every request brings one token, else
    the tcgen05 kernel (head size 64 or 128; windows, chunked masks and soft caps included) or the mma.sync tiled kernel.

    ``rope`` (only where ``fuses_rope``): queries and keys of ``qkv`` are not rotated yet and the newest keys
    and values not yet in their pages; the decode kernel does both.

    ``gate``: a view of ``qkv`` [N, n_q * D]; the output is multiplied by its sigmoid, inside the attention kernel
    except behind the tcgen05 prefill kernel, where `sigmoid_gate` follows.

    ``sinks`` (float32 [n_q]): one more term ``exp(sinks[h])`` in the softmax's denominator of head h; decode steps of
    such layers run the cp.async kernel."""
    if rope is not None and not (qkv.dtype == torch.bfloat16 and ctx.is_decode_only):
        raise KernelError("only bfloat16 decode steps rotate inside the attention kernel")
    if qkv.dtype == torch.float32:
        tile_req, tile_q0 = ctx.query_tiles(16)
        paged_attention_simt(qkv, qkv.shape[1], out, kv, block_tables, tile_req, tile_q0, ctx.q_start,
                             ctx.seq_lens, n_q, n_kv, head_dim, scale, window, chunk, gate, softcap, sinks)
        return
    group = n_q // n_kv
    if ctx.is_decode_only:
        static = ctx.extras.get("static_max_seq_len")  # fixed when the step is captured
        longest = static or ctx.max_seq_len
        wide = ctx.extras.get("decode_wide", False) if static else is_long_context(ctx.max_seq_len)
        wide = bool(wide) and tcgen05_attention_fits(head_dim, n_q, n_kv, kv.shape[3], 0) and sinks is None
        slices = decode_slices(ctx.num_requests, n_kv, group, min(longest, window or chunk or longest), wide,
                               sm_count(qkv.device))
        scratch = ctx.extras.get(("decode_scratch", n_q, head_dim))
        paged_attention_decode(qkv, qkv.shape[1], out, kv, block_tables, ctx.q_start, ctx.seq_lens,
                               ctx.num_requests, n_q, n_kv, head_dim, scale, window, slices, scratch, rope,
                               stages=DECODE_RING_STAGES, chunk=chunk, gate=gate, softcap=softcap, sinks=sinks)
        return
    if tcgen05_prefill_fits(head_dim, n_q, n_kv, kv.shape[3]):
        tile_req, tile_tok0 = ctx.query_tiles_longest_first(128 // group)
        key = ("prefill_key_parts", 128 // group, n_kv, window or chunk)
        parts = ctx.extras.get(key)
        if parts is None:  # the same for every layer of the step that sees as far
            parts = ctx.extras[key] = prefill_key_parts(ctx.q_lens_host, ctx.seq_lens_host, 128 // group, n_kv,
                                                        sm_count(qkv.device), window or chunk)
        paged_attention_prefill_tcgen05(qkv, qkv.shape[1], out, kv, block_tables, tile_req, tile_tok0, ctx.q_start,
                                        ctx.seq_lens, n_q, n_kv, head_dim, scale, parts, chunk, window, softcap, sinks)
        if gate is not None:
            sigmoid_gate(out, gate)
        return
    tile_req, tile_row0 = ctx.query_tiles(64, group)
    paged_attention_prefill(qkv, qkv.shape[1], out, kv, block_tables, tile_req, tile_row0, ctx.q_start,
                            ctx.seq_lens, n_q, n_kv, head_dim, scale, window, chunk, gate, softcap, sinks)


# --------------------------------------------------------------------------- sampling

def argmax(logits: torch.Tensor, with_status: bool = False) -> torch.Tensor:
    """Index of the largest value of each row of float32 ``logits`` [M, V]; the lowest index wins ties.

    ``with_status``: the result has M + 1 elements, the last being the device error word as it stood when the
    kernel ran (``raise_for_status`` reads it on the host), so that the copy that fetches the tokens also tells
    whether a kernel of the step flagged anything."""
    _need(logits, torch.float32, "logits")
    m, v = logits.shape
    out = torch.empty(m + int(with_status), dtype=torch.int32, device=logits.device)
    scratch = torch.empty(m * 32, dtype=torch.int64, device=logits.device)  # one packed word per (row, chunk)
    status = error_word(logits.device).data_ptr() if with_status else None
    _check(ops_library().ss_argmax(logits.data_ptr(), out.data_ptr(), m, v, logits.stride(0), scratch.data_ptr(),
                                   status, _stream()), "argmax")
    _launches[0] += 1  # two kernels
    return out


def sample(logits: torch.Tensor, *, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, penalty: torch.Tensor, seeds: torch.Tensor, draws: torch.Tensor,
           slots: torch.Tensor | None = None, seen: torch.Tensor | None = None,
           with_status: bool = False) -> torch.Tensor:
    """One token per row of float32 ``logits`` [M, V] with per-row parameters (device tensors [M]):
    repetition penalty (needs ``seen`` int32 [slots, ceil(V/32)] and ``slots``), temperature (0 = arg-max),
    top-k (-1 off), top-p, min-p, then a Gumbel-max draw keyed by (seed, draw index).  ``with_status`` as in
    ``argmax``."""
    _need(logits, torch.float32, "logits")
    m, v = logits.shape
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                        ("top_p", top_p, torch.float32), ("min_p", min_p, torch.float32),
                        ("penalty", penalty, torch.float32), ("seeds", seeds, torch.int64),
                        ("draws", draws, torch.int64)):
        _need(t, dt, name)
        if t.numel() != m:
            raise KernelError(f"{name} must hold one value per row")
    seen_words = 0
    if seen is not None:
        _need(seen, torch.int32, "seen")
        _need(slots, torch.int32, "slots")
        seen_words = seen.shape[1]
        if seen_words * 32 < v:
            raise KernelError("the seen-token mask is narrower than the vocabulary")
    out = torch.empty(m + int(with_status), dtype=torch.int32, device=logits.device)
    status = error_word(logits.device).data_ptr() if with_status else None
    _check(ops_library().ss_sample(logits.data_ptr(), logits.stride(0), out.data_ptr(), temperature.data_ptr(),
                                   top_k.data_ptr(), top_p.data_ptr(), min_p.data_ptr(), penalty.data_ptr(),
                                   seeds.data_ptr(), draws.data_ptr(), _ptr(seen), seen_words,
                                   _ptr(slots) if seen is not None else None, m, v, status, _stream()), "sample")
    return out


def mark_seen(seen_row: torch.Tensor, token_ids: torch.Tensor, vocab: int) -> None:
    """Set the bits of ``token_ids`` (int32) in one request's row of the seen-token mask."""
    _need(seen_row, torch.int32, "seen row")
    _need(token_ids, torch.int32, "token_ids")
    _check(ops_library().ss_mark_seen(seen_row.data_ptr(), token_ids.data_ptr(), token_ids.numel(), vocab,
                                      _stream()), "mark_seen")


# --------------------------------------------------------------------------- tensor-core matrix product

_GEMM_COUNTERS = 8192
_GEMM_SCRATCH_FLOATS = 8 * 1024 * 1024


def _gemm_workspace(device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    """Split-K scratch (partial tiles) and per-tile counters; the counters are zero between calls."""
    key = f"gemm_ws{device}"
    ws = _state.get(key)
    if ws is None:
        ws = (torch.empty(_GEMM_SCRATCH_FLOATS, dtype=torch.float32, device=device),
              torch.zeros(_GEMM_COUNTERS, dtype=torch.int32, device=device))
        _state[key] = ws
    return ws  # type: ignore[return-value]


@dataclasses.dataclass
class PendingNorm:
    """``weight * round(stream * rsqrt(mean(stream^2) + eps))`` that has not been computed: the stream is complete
    (the branch in front has been added), ``scaled`` holds ``round(weight * stream)`` in bfloat16 and ``squares``
    [tokens, tiles] the sums of the stream's squares per tile of 128 features.  `linear` and `gate_up_swiglu` take it
    in place of the activations: with few bfloat16 tokens the product runs on ``scaled`` and multiplies every
    token's output by its ``rsqrt(...)`` at the end (the scale does not depend on the feature, so it commutes with
    the product; the activations are then rounded once instead of twice).  Everything else calls
    ``materialize()``, the norm kernel on the stream."""
    stream: torch.Tensor
    scaled: torch.Tensor
    squares: torch.Tensor
    weight: torch.Tensor
    eps: float
    dtype: torch.dtype
    # hyper-connected streams: ``stream`` is [tokens, S, hidden] and the norm is that of sum_t w_in[t] * stream t
    # (``w_in`` None: the plain sum); ``scaled`` and ``squares`` describe that sum
    w_in: torch.Tensor | None = None

    @property
    def shape(self) -> torch.Size:
        return self.scaled.shape

    @property
    def device(self) -> torch.device:
        return self.stream.device

    def materialize(self) -> torch.Tensor:
        if self.stream.dim() == 3:
            return hc_norm(self.stream, None, None, None, self.w_in, self.weight, self.eps, self.dtype)
        return add_rmsnorm(self.stream, None, self.weight, self.eps, self.dtype)


def takes_pending_norm(x: "torch.Tensor | PendingNorm", features: int, swiglu: bool = False) -> bool:
    """Whether the product of ``x`` with a [features, K] weight applies the norm's scale inside the kernel: the
    streaming kernel of decode steps, or the two-SM kernel of long prompt portions."""
    if not isinstance(x, PendingNorm) or x.dtype != torch.bfloat16:
        return False
    sms = sm_count(x.device)
    if x.shape[0] <= CLUSTER_BATCH and streams_weights(x.shape[0], features, x.shape[1], sms):
        return True
    if swiglu:
        return x.shape[1] % 8 == 0 and many_tokens_swiglu_fits(x.shape[0], features, sms)
    return many_tokens_fits(x.shape[0], features, x.shape[1], sms)


def gemm_plan(tokens: int, features: int, k: int, sms: int | None = None) -> tuple[bool, int, int]:
    """(swapped, tile width, K slices) for ``x[tokens, k] @ w[features, k].T`` on ``sms`` multiprocessors."""
    return _gemm_plan(tokens, features, k, sms or sm_count())


@functools.lru_cache(maxsize=None)
def _gemm_plan(tokens: int, features: int, k: int, sms: int) -> tuple[bool, int, int]:
    k_iters = (k + 63) // 64
    if tokens <= 64:
        bn = 16 if tokens <= 16 else (32 if tokens <= 32 else 64)
        tiles = (features + 127) // 128
        # at most 8 slices: they then form one thread-block cluster and are added through shared memory
        slices = max(1, min(k_iters, (2 * sms + tiles - 1) // tiles if tiles < sms else 1, 8))
        # the widest tile leaves room for two blocks per SM, and clusters do not pack an SM's last slot: stay
        # within one wave of blocks (36 tiles x 8 slices ran as two waves: 18.1 us against 13.2 with 7 slices)
        while bn == 64 and slices > 1 and tiles * slices > sms + (3 * sms) // 4:
            slices -= 1
        return True, bn, slices
    bn = 256 if features >= 256 else (128 if features >= 128 else (64 if features >= 64 else (32 if features >= 32 else 16)))
    return False, bn, 1


def gemm_tcgen05(x: "torch.Tensor | PendingNorm", weight: torch.Tensor, bias: torch.Tensor | None = None,
                 out_dtype: torch.dtype | None = None, plan: tuple[bool, int, int] | None = None,
                 swiglu: bool = False, to_stream: tuple[torch.Tensor, torch.Tensor] | None = None,
                 glu: tuple[float, float, float] | None = None, hc: "np.ndarray | None" = None):
    """``x @ weight.T + bias`` for bfloat16 ``x`` [tokens, K] and ``weight`` [features, K] on the tcgen05 tensor
    cores (TMA-fed, accumulator in tensor memory); output bfloat16 or float32.  K must be a multiple of 8.

    ``swiglu`` (at most 64 tokens, features a multiple of 128): the weight's rows alternate 64 gate and 64 up
    features; the result is ``silu(gate) * up`` with features / 2 columns, formed in the product's epilogue.

    ``glu`` = (alpha, limit, shift) with ``swiglu``: the fused unit is `glu_limited`'s instead of SwiGLU.
    ``hc`` with ``to_stream``: the stream is [tokens, S, features], S hyper-connected streams (at most 4), and ``hc`` a
    float32 host array of S * S + 2 S values, mix [from, to], out, in: the product is written into the streams as
    `hc_norm` writes a branch output, and what comes back describes ``sum_t in[t] * stream t``.

    ``to_stream`` = (float32 stream [tokens, features], weights of the norm behind it), where `adds_to_stream`:
    the product, rounded to bfloat16, is added to the stream in place instead of being returned, and the function
    returns (round(norm weights * new stream) in bfloat16, sums of squares [tokens, features / 128]).
    ``x`` may be a `PendingNorm` (at most 16 tokens): the product runs on its ``scaled`` and applies the scale of
    every token in the epilogue."""
    pending = x if isinstance(x, PendingNorm) else None
    if pending is not None:
        if pending.dtype != torch.bfloat16:
            raise KernelError("a pending norm feeds the tensor-core product only in bfloat16")
        x = pending.scaled
    _need(x, torch.bfloat16, "x")
    _need(weight, torch.bfloat16, "weight")
    tokens, k = x.shape
    features = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"weight {tuple(weight.shape)} does not match x {tuple(x.shape)}")
    if k % 8 != 0:
        raise KernelError(f"the tensor-core matrix product needs K to be a multiple of 8, got {k}")
    out_dtype = out_dtype or torch.bfloat16
    if swiglu and (tokens > 64 or features % 128):
        raise KernelError("the fused SwiGLU epilogue takes at most 64 tokens and a multiple of 128 weight rows")
    out_shape = (tokens, features // 2 if swiglu else features)
    out = None if to_stream is not None else torch.empty(out_shape, dtype=out_dtype, device=x.device)
    if tokens == 0:
        return out
    bias_f32 = 0
    if bias is not None:
        _need(bias, None, "bias")
        bias_f32 = int(bias.dtype == torch.float32)
        if bias.numel() != features or bias.dtype not in (torch.float32, torch.bfloat16):
            raise KernelError("bias has the wrong size or dtype")
    swapped, bn, slices = plan or gemm_plan(tokens, features, k, sm_count(x.device))
    partial = counters = None
    if slices > 1 and not (swapped and slices <= 8 and tokens <= bn):
        partial, counters = _gemm_workspace(x.device)
        tiles = ((features if swapped else tokens) + 127) // 128 * (((tokens if swapped else features) + bn - 1) // bn)
        if tiles > _GEMM_COUNTERS or tiles * slices * bn * 128 > _GEMM_SCRATCH_FLOATS:
            raise KernelError("split-K workspace too small for this problem")
    a, b = (weight, x) if swapped else (x, weight)
    if to_stream is not None:
        stream, norm_weight = to_stream
        _need(stream, torch.float32, "stream")
        _need(norm_weight, None, "norm weight")
        n_streams = 0
        if hc is not None:
            n_streams = stream.shape[1] if stream.dim() == 3 else 0
            if not 1 <= n_streams <= 4 or hc.dtype != np.float32 or hc.size != n_streams * (n_streams + 2) \
                    or not hc.flags["C_CONTIGUOUS"]:
                raise KernelError("hyper-connected streams: [tokens, S <= 4, features] and S * S + 2 S float32 weights")
        stream_shape = (tokens, n_streams, features) if n_streams else out_shape
        if (swiglu or pending is not None or out_dtype != torch.bfloat16 or tuple(stream.shape) != stream_shape
                or not (swapped and 2 <= slices <= 8 and tokens <= bn) or features % 128
                or norm_weight.numel() != features or norm_weight.dtype not in (torch.float32, torch.bfloat16)):
            raise KernelError("a product into the stream needs its plain bfloat16 output, K slices in a cluster, a "
                              "width in steps of 128 and a stream of its shape")
        scaled = torch.empty((tokens, features), dtype=torch.bfloat16, device=x.device)
        squares = torch.empty((tokens, features // 128), dtype=torch.float32, device=x.device)
        if n_streams:
            rc = gemm_library().ss_gemm_tc5_to_streams(a.data_ptr(), b.data_ptr(), _ptr(bias), bias_f32, a.shape[0],
                                                       b.shape[0], k, k, k, bn, slices, stream.data_ptr(), n_streams,
                                                       hc.ctypes.data, squares.data_ptr(), scaled.data_ptr(),
                                                       norm_weight.data_ptr(), int(norm_weight.dtype == torch.float32),
                                                       error_word(x.device).data_ptr(), _stream())
            _check(rc, "gemm_tcgen05 into hyper-connected streams")
            return scaled, squares
        rc = gemm_library().ss_gemm_tc5_to_stream(a.data_ptr(), b.data_ptr(), _ptr(bias), bias_f32, a.shape[0], b.shape[0],
                                                  k, k, k, bn, slices, stream.data_ptr(), squares.data_ptr(),
                                                  scaled.data_ptr(), norm_weight.data_ptr(),
                                                  int(norm_weight.dtype == torch.float32),
                                                  error_word(x.device).data_ptr(), _stream())
        _check(rc, "gemm_tcgen05 into the stream")
        return scaled, squares
    if pending is not None:
        if not swapped or bn != 16 or pending.weight.numel() != k or pending.squares.shape[0] != tokens:
            raise KernelError("a pending norm feeds the swapped product of at most 16 tokens, over the stream's whole width")
        if glu is not None:
            if not swiglu:
                raise KernelError("the constants of a gated unit come with the fused gate/up epilogue")
            rc = gemm_library().ss_gemm_tc5_scaled_glu(a.data_ptr(), b.data_ptr(), pending.squares.data_ptr(),
                                                       pending.squares.shape[1], float(pending.eps), _ptr(bias), bias_f32,
                                                       out.data_ptr(), a.shape[0], tokens, k, k, k, out.shape[1], bn,
                                                       int(out_dtype == torch.float32), slices, float(glu[0]),
                                                       float(glu[1]), float(glu[2]), _ptr(partial), _ptr(counters),
                                                       error_word(x.device).data_ptr(), _stream())
            _check(rc, "gemm_tcgen05 with a gated unit behind a pending norm")
            return out
        rc = gemm_library().ss_gemm_tc5_scaled(a.data_ptr(), b.data_ptr(), pending.squares.data_ptr(),
                                               pending.squares.shape[1], float(pending.eps), _ptr(bias), bias_f32,
                                               out.data_ptr(), a.shape[0], tokens, k, k, k, out.shape[1], bn,
                                               int(out_dtype == torch.float32), slices, int(swiglu), _ptr(partial),
                                               _ptr(counters), error_word(x.device).data_ptr(), _stream())
        _check(rc, "gemm_tcgen05 behind a pending norm")
        return out
    if glu is not None:
        if not swiglu:
            raise KernelError("the constants of a gated unit come with the fused gate/up epilogue")
        rc = gemm_library().ss_gemm_tc5_glu(a.data_ptr(), b.data_ptr(), _ptr(bias), bias_f32, out.data_ptr(), a.shape[0],
                                            b.shape[0], k, k, k, out.shape[1], bn, int(swapped),
                                            int(out_dtype == torch.float32), slices, float(glu[0]), float(glu[1]),
                                            float(glu[2]), _ptr(partial), _ptr(counters),
                                            error_word(x.device).data_ptr(), _stream())
        _check(rc, "gemm_tcgen05 with a gated unit")
        return out
    rc = gemm_library().ss_gemm_tc5(a.data_ptr(), b.data_ptr(), _ptr(bias), bias_f32, out.data_ptr(), a.shape[0],
                                    b.shape[0], k, k, k, out.shape[1], bn, int(swapped), int(out_dtype == torch.float32),
                                    slices, int(swiglu), _ptr(partial), _ptr(counters),
                                    error_word(x.device).data_ptr(), _stream())
    _check(rc, "gemm_tcgen05")
    return out


def gemm_tcgen05_many(x: "torch.Tensor | PendingNorm", weight: torch.Tensor, bias: torch.Tensor | None = None,
                      out_dtype: torch.dtype | None = None, swiglu: bool = False, tile_cols: int = 0,
                      to_stream: tuple[torch.Tensor, torch.Tensor] | None = None,
                      glu: tuple[float, float, float] | None = None):
    """``x @ weight.T + bias`` for many rows of ``x`` (prompt portions) on the tcgen05 tensor cores: a persistent
    kernel, one block per SM, the blocks in pairs (``tcgen05.mma.cta_group::2``: each block of a pair loads half
    of A and half of B) that compute tiles of 256 rows with the accumulator double-buffered in tensor memory, so
    that the epilogue of a tile overlaps the products of the next.  ``tile_cols``: the tiles' width, a multiple
    of 16 up to 256; 0 lets the launcher take the width whose tiles fill whole rounds of the pairs of SMs best.
    ``swiglu``: the weight's rows alternate 64 gate and 64 up features; the result is ``silu(gate) * up`` with
    features / 2 columns (tiles of 256 columns).  ``to_stream`` and a `PendingNorm` for ``x``: as in
    `gemm_tcgen05` (features a multiple of 16; the sums of squares come per tile of the chosen width)."""
    pending = x if isinstance(x, PendingNorm) else None
    if pending is not None:
        if pending.dtype != torch.bfloat16:
            raise KernelError("a pending norm feeds the tensor-core product only in bfloat16")
        x = pending.scaled
    _need(x, torch.bfloat16, "x")
    _need(weight, torch.bfloat16, "weight")
    tokens, k = x.shape
    features = weight.shape[0]
    if weight.shape[1] != k or k % 8 != 0:
        raise KernelError("the tensor-core matrix product needs matching K, a multiple of 8")
    out_dtype = out_dtype or torch.bfloat16
    if swiglu and (features % 128 or out_dtype != torch.bfloat16 or (features // 2) % 8):
        raise KernelError("the fused SwiGLU epilogue takes a multiple of 128 weight rows and writes bfloat16")
    out_shape = (tokens, features // 2 if swiglu else features)
    out = None if to_stream is not None else torch.empty(out_shape, dtype=out_dtype, device=x.device)
    if tokens == 0:
        return out
    bias_f32 = 0
    if bias is not None:
        _need(bias, None, "bias")
        bias_f32 = int(bias.dtype == torch.float32)
        if bias.numel() != features or bias.dtype not in (torch.float32, torch.bfloat16):
            raise KernelError("bias has the wrong size or dtype")
    if to_stream is not None:
        stream, norm_weight = to_stream
        _need(stream, torch.float32, "stream")
        _need(norm_weight, None, "norm weight")
        if (swiglu or pending is not None or out_dtype != torch.bfloat16 or tuple(stream.shape) != out_shape or features % 16
                or norm_weight.numel() != features or norm_weight.dtype not in (torch.float32, torch.bfloat16)):
            raise KernelError("a product into the stream needs its plain bfloat16 output, a width in steps of 16 and a "
                              "stream of its shape")
        width = tile_cols or gemm_library().ss_gemm_tc5_many_tile_cols(tokens, features, 0)
        scaled = torch.empty((tokens, features), dtype=torch.bfloat16, device=x.device)
        squares = torch.empty((tokens, (features + width - 1) // width), dtype=torch.float32, device=x.device)
        rc = gemm_library().ss_gemm_tc5_many_to_stream(x.data_ptr(), weight.data_ptr(), _ptr(bias), bias_f32, tokens,
                                                       features, k, k, k, width, stream.data_ptr(), squares.data_ptr(),
                                                       scaled.data_ptr(), norm_weight.data_ptr(),
                                                       int(norm_weight.dtype == torch.float32),
                                                       error_word(x.device).data_ptr(), _stream())
        _check(rc, "gemm_tcgen05_many into the stream")
        return scaled, squares
    if pending is not None:
        if pending.weight.numel() != k or pending.squares.shape[0] != tokens:
            raise KernelError("a pending norm feeds a product over the stream's whole width")
        rc = gemm_library().ss_gemm_tc5_many_scaled(x.data_ptr(), weight.data_ptr(), pending.squares.data_ptr(),
                                                    pending.squares.shape[1], float(pending.eps), _ptr(bias), bias_f32,
                                                    out.data_ptr(), tokens, features, k, k, k, out.shape[1],
                                                    int(out_dtype == torch.float32), int(swiglu), tile_cols,
                                                    error_word(x.device).data_ptr(), _stream())
        _check(rc, "gemm_tcgen05_many behind a pending norm")
        return out
    if glu is not None:
        if not swiglu:
            raise KernelError("the constants of a gated unit come with the fused gate/up epilogue")
        rc = gemm_library().ss_gemm_tc5_many_glu(x.data_ptr(), weight.data_ptr(), _ptr(bias), bias_f32, out.data_ptr(),
                                                 tokens, features, k, k, k, out.shape[1], float(glu[0]), float(glu[1]),
                                                 float(glu[2]), error_word(x.device).data_ptr(), _stream())
        _check(rc, "gemm_tcgen05_many with a gated unit")
        return out
    rc = gemm_library().ss_gemm_tc5_many(x.data_ptr(), weight.data_ptr(), _ptr(bias), bias_f32, out.data_ptr(), tokens,
                                         features, k, k, k, out.shape[1], int(out_dtype == torch.float32), int(swiglu),
                                         tile_cols, error_word(x.device).data_ptr(), _stream())
    _check(rc, "gemm_tcgen05_many")
    return out


# From this many tokens a bfloat16 projection whose 256 x 256 output tiles make at least a round and a half of the
# pairs of SMs, and whose K is deep enough for a tile's first loads and its epilogue to be a small part of it
# (``many_tokens_fits``), runs the persistent two-SM kernel.  Against the library (us, ours / library) at 2,048 tokens: 7B sizes q/k/v 49.6 / 45.1, o 41.6-47.7 /
# 45.4-52.8, down 191.9-198.2 / 191.6-208.7; 14B sizes 109.4 / 114.6, 79.7 / 77.0, 200.3 / 207.2; a whole 2,048-token
# prefill of the 7B shape takes 22.1 to 25.5 ms either way (the GPU sits at its power cap), and its first call 35
# ms instead of 160.  With fewer tokens or smaller weights there are too few 256-row tiles for the pairs of SMs and
# the library, which splits K, wins: 1,024 tokens at 14B sizes by up to 18 %, 0.5B and 1.5B sizes at any number
# of tokens by up to 50 %, 512 tokens and below by 1.3 to 2 times.  (Cutting K into parts inside this kernel,
# with the parts' sums meeting in scratch memory, was tried for those cases and did not beat narrower tiles.)
MANY_TOKENS = 2048
MANY_K_STEPS = 32  # 64-wide K steps a tile must have (2,048 columns)


def many_tokens_fits(tokens: int, features: int, k: int, sms: int | None = None) -> bool:
    """Where the persistent two-SM tcgen05 kernel is the product of a prompt portion (see the measurements above):
    at the 7B and 14B layer sizes from 2,048 tokens (112 to 224 tiles on 74 pairs), not at the 0.5B and 1.5B sizes
    (40 to 48 tiles, K of 896 and 1,536)."""
    if tokens < MANY_TOKENS or k % 8 != 0 or k < 64 * MANY_K_STEPS:
        return False
    tiles = ((tokens + 255) // 256) * ((features + 255) // 256)
    return 4 * tiles >= 3 * (sms or sm_count())  # a round and a half of the sms / 2 pairs


SMALL_BATCH = 64  # up to this many tokens a projection may stream its weights through the tcgen05 kernel
# ... when its 128-row weight tiles are at least as many as the SMs (no K slices needed)
CLUSTER_BATCH = 16  # ... or, up to this many tokens, whatever its size (K slices added inside a cluster)
DEEP_K = 8192  # ... or when K is at least this deep: every block then streams enough to pay for its set-up


def streams_weights(tokens: int, features: int, k: int, sms: int | None = None) -> bool:
    """True where the hand-written tcgen05 kernel is the faster way to run a bfloat16 projection.  Measured
    on the 7B shape inside a decode step: with enough weight tiles to give every SM one (gate/up, LM head) it
    wins up to 64 tokens (43 us against the library's 46.5 us at 8 tokens); the smaller products (q/k/v, o,
    down), whose K range is cut into slices that a thread-block cluster adds, win up to 16 tokens (a step of
    8 requests: 3.18 ms against 3.41 ms with the library's split-K kernels); at 32 and 64 tokens only the
    down product still wins (25.6 and 28.0 us against 29.1 and 30.8), q/k/v and o lose by 1 to 9 us."""
    if k % 8 != 0 or tokens > SMALL_BATCH:
        return False
    return tokens <= CLUSTER_BATCH or (features + 127) // 128 >= (sms or sm_count()) or k >= DEEP_K


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
           out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """A projection ``x @ weight.T + bias``.

    float32 runs the CUDA-core kernel (no reduced-precision matrix mode).  bfloat16 with few tokens (decode
    steps) and a large weight runs the hand-written tcgen05 kernel, which streams the weights once and
    overlaps its first fetches with the kernel before it; from ``MANY_TOKENS`` tokens (prompt portions) and with
    enough output tiles (``many_tokens_fits``) the persistent two-SM tcgen05 kernel; everything else runs the
    library matrix product, as the reference's
    nn.Linear does (slipstream/models/layers/attention.py:132-135).  ``x`` may be a `PendingNorm`."""
    if isinstance(x, PendingNorm):
        if not takes_pending_norm(x, weight.shape[0]):
            x = x.materialize()
        elif x.shape[0] <= CLUSTER_BATCH:
            return gemm_tcgen05(x, weight, bias, out_dtype)
        else:
            return gemm_tcgen05_many(x, weight, bias, out_dtype)
    if x.dtype == torch.float32:
        return gemm_simt(x, weight, bias, out_dtype)
    sms = sm_count(x.device)
    if streams_weights(x.shape[0], weight.shape[0], x.shape[1], sms):
        return gemm_tcgen05(x, weight, bias, out_dtype)
    if many_tokens_fits(x.shape[0], weight.shape[0], x.shape[1], sms):
        return gemm_tcgen05_many(x, weight, bias, out_dtype)
    if out_dtype is None or out_dtype == x.dtype:
        if bias is not None:
            return torch.addmm(bias, x, weight.t())
        return torch.mm(x, weight.t())
    out = torch.mm(x, weight.t(), out_dtype=out_dtype)
    if bias is not None:
        out += bias
    return out


def adds_to_stream(tokens: int, features: int, k: int, sms: int | None = None) -> bool:
    """True where a bfloat16 projection can add its output to the float32 stream itself and prepare the norm
    behind it: the streaming tcgen05 kernel with its K slices as a thread-block cluster (decode steps), a width in
    steps of 128."""
    sms = sms or sm_count()
    if not _state.get("norm_rides_along", True):
        return False
    if _state.get("norm_rides_along_long", False) and features % 16 == 0 and many_tokens_fits(tokens, features, k, sms):
        return True  # the two-SM kernel of long prompt portions: every thread of its epilogue has a row
    if features % 128 != 0 or tokens > CLUSTER_BATCH or not streams_weights(tokens, features, k, sms):
        return False
    swapped, bn, slices = gemm_plan(tokens, features, k, sms)
    return swapped and 2 <= slices <= 8 and tokens <= bn


def set_norm_fusion(enabled: bool, long_portions: bool = False) -> None:
    """Whether `linear_add_rmsnorm` may leave the norm to the products around it (on by default; off for
    comparisons).  ``long_portions``: also in the two-SM kernel of prompt portions from 2,048 tokens.  That is off
    unless asked for, by measurement at the 7B sizes: the o and down products with the add inside take 71 and 225
    us, as long as the product followed by the norm kernel (72 and 225: the read-modify-write of the stream from
    an epilogue that holds a row per thread costs what the norm kernel cost), q/k/v and gate/up with the scale
    in their epilogue take what they took, and a whole 2,048-token step 21.67 ms against 21.5 to 21.6."""
    _state["norm_rides_along"] = bool(enabled)
    _state["norm_rides_along_long"] = bool(enabled and long_portions)


def linear_add_rmsnorm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, residual: torch.Tensor,
                       norm_weight: torch.Tensor, eps: float, out_dtype: torch.dtype) -> "torch.Tensor | PendingNorm":
    """``residual += x @ weight.T + bias`` (float32 stream, in place; the branch output rounded to the compute dtype
    first), then the RMS norm of the stream times ``norm_weight``: a branch's last projection with the add and the
    norm that follow it.  With few bfloat16 tokens the projection adds to the stream in its epilogue and the
    norm comes back as a `PendingNorm`, to be finished by the next product (no norm kernel); everything
    else is `linear` followed by `add_rmsnorm`."""
    if x.shape[0] > 0 and x.dtype == torch.bfloat16 and out_dtype == torch.bfloat16 \
            and residual.shape == (x.shape[0], weight.shape[0]) \
            and norm_weight.numel() == weight.shape[0] \
            and adds_to_stream(x.shape[0], weight.shape[0], x.shape[1], sm_count(x.device)):
        product = gemm_tcgen05 if x.shape[0] <= SMALL_BATCH else gemm_tcgen05_many
        scaled, squares = product(x, weight, bias, to_stream=(residual, norm_weight))
        return PendingNorm(residual, scaled, squares, norm_weight, eps, out_dtype)
    return add_rmsnorm(residual, linear(x, weight, bias), norm_weight, eps, out_dtype)


def linear_hc_rmsnorm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, streams: torch.Tensor,
                      mix: torch.Tensor, w_out: torch.Tensor, w_in: torch.Tensor | None, hc_host: "np.ndarray | None",
                      norm_weight: torch.Tensor, eps: float, out_dtype: torch.dtype) -> "torch.Tensor | PendingNorm":
    """`linear_add_rmsnorm` for hyper-connected streams [tokens, S, hidden]: ``y = x @ weight.T + bias`` is written
    into the streams with the branch's ``mix`` and ``w_out``, and the norm of ``sum_t w_in[t] * stream t`` comes back
    (see `hc_norm`).  With few bfloat16 tokens and at most 4 streams the product does the write in its epilogue
    (``hc_host``: the same weights as a float32 host array, mix, out, in) and the norm comes back as a
    `PendingNorm`; everything else is `linear` followed by `hc_norm`."""
    tokens, n_streams, hidden = streams.shape
    if hc_host is not None and tokens > 0 and n_streams <= 4 and x.dtype == torch.bfloat16 and out_dtype == torch.bfloat16 \
            and weight.shape[0] == hidden and norm_weight.numel() == hidden and x.shape[0] <= SMALL_BATCH \
            and adds_to_stream(tokens, hidden, x.shape[1], sm_count(x.device)):
        scaled, squares = gemm_tcgen05(x, weight, bias, to_stream=(streams, norm_weight), hc=hc_host)
        return PendingNorm(streams, scaled, squares, norm_weight, eps, out_dtype, w_in=w_in)
    return hc_norm(streams, linear(x, weight, bias), mix, w_out, w_in, norm_weight, eps, out_dtype)


def many_tokens_swiglu_fits(tokens: int, features: int, sms: int | None = None) -> bool:
    """Where the persistent tcgen05 kernel with its fused SwiGLU epilogue is at least as fast as the library
    product followed by the SwiGLU kernel: enough 256 x 256 tiles to keep every pair of SMs busy for several
    rounds (2,048 tokens x 37,888 features: 347 us against 348 + 40 us, and no [tokens, 2 I] intermediate; 1,024
    tokens: 205 against 179 + 20; 512 tokens: 108 against 95 + 10, where the library stays).  Without an epilogue
    to fuse, the library product is as fast as ours or up to 10 % faster, and stays."""
    return ((tokens + 255) // 256) * ((features + 255) // 256) >= 4 * (sms or sm_count())


def gate_up_swiglu(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, block: int) -> torch.Tensor:
    """``silu(x @ Wg.T + bg) * (x @ Wu.T + bu)`` where ``weight`` [2 I, K] holds gate and up rows alternating in
    runs of ``block``.  Small bfloat16 batches with runs of 64 do it in one kernel.  ``x`` may be a `PendingNorm`."""
    if isinstance(x, PendingNorm):
        if block == 64 and weight.shape[0] % 128 == 0 and takes_pending_norm(x, weight.shape[0], swiglu=True):
            if x.shape[0] <= CLUSTER_BATCH:
                return gemm_tcgen05(x, weight, bias, swiglu=True)
            return gemm_tcgen05_many(x, weight, bias, swiglu=True)
        x = x.materialize()
    if x.dtype == torch.bfloat16 and block == 64 and weight.shape[0] % 128 == 0 and x.shape[1] % 8 == 0:
        sms = sm_count(x.device)
        if streams_weights(x.shape[0], weight.shape[0], x.shape[1], sms):
            return gemm_tcgen05(x, weight, bias, swiglu=True)
        if many_tokens_swiglu_fits(x.shape[0], weight.shape[0], sms):
            return gemm_tcgen05_many(x, weight, bias, swiglu=True)
    return swiglu(linear(x, weight, bias), block=block)


def gate_up_glu(x: "torch.Tensor | PendingNorm", weight: torch.Tensor, bias: torch.Tensor | None, block: int,
                alpha: float, limit: float, shift: float) -> torch.Tensor:
    """`gate_up_swiglu` with the gated unit of `glu_limited` (a steeper sigmoid, clamped inputs, a shifted up
    branch).  Where `gate_up_swiglu` forms SwiGLU in the product's epilogue (small bfloat16 batches, long prompt
    portions; runs of 64) this does the same with the unit's constants; everything else is the stacked product
    followed by the activation kernel."""
    if isinstance(x, PendingNorm):
        if (block == 64 and weight.shape[0] % 128 == 0 and x.shape[0] <= CLUSTER_BATCH
                and takes_pending_norm(x, weight.shape[0], swiglu=True)):
            return gemm_tcgen05(x, weight, bias, swiglu=True, glu=(alpha, limit, shift))
        x = x.materialize()
    if x.dtype == torch.bfloat16 and block == 64 and weight.shape[0] % 128 == 0 and x.shape[1] % 8 == 0:
        sms = sm_count(x.device)
        if streams_weights(x.shape[0], weight.shape[0], x.shape[1], sms):
            return gemm_tcgen05(x, weight, bias, swiglu=True, glu=(alpha, limit, shift))
        if many_tokens_swiglu_fits(x.shape[0], weight.shape[0], sms):
            return gemm_tcgen05_many(x, weight, bias, swiglu=True, glu=(alpha, limit, shift))
    return glu_limited(linear(x, weight, bias), block, alpha, limit, shift)


# --------------------------------------------------------------------------- grouped norm, state-space mixer, routed experts

def group_norm(x: torch.Tensor, weight: torch.Tensor, groups: int, eps: float, out_dtype: torch.dtype, *,
               residual: torch.Tensor | None = None, rows: torch.Tensor | None = None, gate: torch.Tensor | None = None,
               terms: int = 1, extra: torch.Tensor | None = None, want_out: bool = True,
               term_rows: torch.Tensor | None = None) -> torch.Tensor | None:
    """RMS norm in ``groups`` equal consecutive parts of the last axis, each part over its own root mean square
    (``v / sqrt(mean(v^2) + eps)``), times ``weight`` (float32 [hidden]); float32 arithmetic, one rounding.

    ``x`` [N, hidden] in ``out_dtype`` or float32.  ``terms`` > 1: ``x`` is [N, terms, hidden] (float32) and the
    terms are summed first; ``extra`` [N, hidden] (``out_dtype``) is added to that sum.  ``term_rows`` (int32
    [N * terms]): ``x`` is [any, hidden] and term k of row r is its row ``term_rows[r * terms + k]``.  ``gate`` (a view [N, hidden]
    with unit inner stride, ``out_dtype``): the input is multiplied by ``silu(gate)`` before the norm.
    ``residual`` (float32 [N, hidden]): the result is ADDED to it in place, and what is returned is the new
    residual rounded to ``out_dtype`` (nothing with ``want_out`` False).  ``rows`` (int32 [M]): only those rows
    of ``x`` are normed and returned."""
    hidden = weight.numel()
    _need(weight, torch.float32, "norm weight")
    if x.dtype not in (out_dtype, torch.float32) or not x.is_cuda or not x.is_contiguous():
        raise KernelError("group_norm takes a contiguous CUDA tensor in the compute dtype or float32")
    if term_rows is not None:
        _need(term_rows, torch.int32, "term_rows")
        if x.dim() != 2 or term_rows.numel() % terms:
            raise KernelError("with term_rows, x must be [rows, hidden] and term_rows hold N * terms entries")
    elif terms > 1 and (x.dim() != 3 or x.shape[1] != terms or x.dtype != torch.float32):
        raise KernelError("with terms, x must be float32 [N, terms, hidden]")
    if x.shape[-1] != hidden or groups < 1 or hidden % groups:
        raise KernelError(f"group_norm: {hidden} features do not split into {groups} groups, or x is of another width")
    n = x.shape[0] if term_rows is None else term_rows.numel() // terms
    n_out = n if rows is None else rows.numel()
    if rows is not None:
        _need(rows, torch.int32, "rows")
        if residual is not None:
            raise KernelError("a selection of rows is not added to the stream")
    if residual is not None:
        _need(residual, torch.float32, "residual")
        if tuple(residual.shape) != (n, hidden):
            raise KernelError("residual does not match x")
    if extra is not None:
        _need(extra, out_dtype, "extra")
    gate_stride = 0
    if gate is not None:
        if gate.dtype != out_dtype or gate.dim() != 2 or gate.stride(1) != 1 or tuple(gate.shape) != (n, hidden):
            raise KernelError("the gate must be [N, hidden] in the compute dtype with unit inner stride")
        gate_stride = gate.stride(0)
    out = torch.empty((n_out, hidden), dtype=out_dtype, device=x.device) if want_out else None
    _check(ops_library().ss_group_norm(x.data_ptr(), int(x.dtype == torch.float32), terms * hidden, int(terms), _ptr(extra),
                                       _ptr(gate), gate_stride, weight.data_ptr(), _ptr(residual), _ptr(out), _ptr(rows),
                                       n_out, hidden, int(groups), float(eps), _code(out_dtype), _stream(), _ptr(term_rows)),
           "group_norm")
    return out


def round_stream(residual: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """The float32 stream as a branch reads it: itself in float32, rounded once in bfloat16."""
    _need(residual, torch.float32, "residual")
    if out_dtype == torch.float32:
        return residual
    out = torch.empty(residual.shape, dtype=torch.bfloat16, device=residual.device)
    _check(ops_library().ss_round_stream(residual.data_ptr(), out.data_ptr(), residual.numel(), _stream()), "round_stream")
    return out


def conv_silu(proj: torch.Tensor, col0: int, channels: int, taps: torch.Tensor, bias: torch.Tensor | None,
              state: torch.Tensor, ctx, plus_input: bool = False, activation: bool = True) -> torch.Tensor:
    """``silu`` of a causal convolution per channel over each request's tokens.  Channel c of a token is
    ``proj[row, col0 + c]``; ``taps`` float32 [channels, T] (the last column multiplies the current token);
    ``state`` float32 [slots, T - 1, channels] holds each request's last T - 1 inputs (zeros for a request that
    starts), is read for the tokens in front of the step and left holding the step's last inputs.  Returns
    [N, channels] in the dtype of ``proj``.  ``plus_input``: the result is ``input + convolution`` with no activation
    instead (a convolution laid over a branch's input).  ``activation`` False: the convolution (with its bias) as it
    is."""
    if plus_input and not activation:
        raise KernelError("conv_silu: plus_input has no activation already")
    _need(proj, None, "projection")
    _need(taps, torch.float32, "taps")
    _need(state, torch.float32, "convolution state")
    n_taps = taps.shape[1]
    if bias is not None:
        _need(bias, torch.float32, "convolution bias")
    if tuple(taps.shape) != (channels, n_taps) or tuple(state.shape[1:]) != (max(n_taps - 1, 0), channels):
        raise KernelError("taps must be [channels, T] and the state [slots, T - 1, channels]")
    if col0 < 0 or col0 + channels > proj.shape[1] or n_taps > 8:
        raise KernelError("the convolution's channels lie outside the projection, or it has more than 8 taps")
    n = proj.shape[0]
    out = torch.empty((n, channels), dtype=proj.dtype, device=proj.device)
    _check(ops_library().ss_conv_silu(proj.data_ptr(), proj.stride(0), int(col0), taps.data_ptr(), _ptr(bias),
                                      state.data_ptr(), out.data_ptr(), ctx.q_start.data_ptr(), ctx.seq_lens.data_ptr(),
                                      ctx.state_slots.data_ptr(), ctx.num_requests, n, channels, n_taps, state.shape[0],
                                      int(ctx.is_decode_only), _code(proj.dtype), error_word(proj.device).data_ptr(),
                                      _stream(), 1 if plus_input else (0 if activation else 2)), "conv_silu")
    if not ctx.is_decode_only and n_taps > 1:
        _launches[0] += 1  # the state's update is a launch of its own
    return out


def ssm_scan(xbc: torch.Tensor, dt: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor,
             state: torch.Tensor, ctx, heads: int, groups: int, head_dim: int, state_dim: int) -> torch.Tensor:
    """The diagonal state-space recurrence over each request's tokens, continued from and left in ``state``
    (float32 [slots, heads, head_dim, state_dim]).  ``xbc`` [N, heads * head_dim + 2 * groups * state_dim] holds x, then
    B, then C; ``dt`` [N, heads] is a view of the raw step sizes (unit inner stride).  Per head h (group
    ``h // (heads / groups)``): ``dt' = softplus(dt + dt_bias[h])``, ``S <- exp(-exp(a_log[h]) dt') S + dt' B x^T``,
    ``y = S^T C + d_skip[h] x``.  Returns y float32 [N, heads * head_dim]."""
    _need(xbc, None, "x, B and C")
    for name, t in (("dt_bias", dt_bias), ("a_log", a_log), ("d_skip", d_skip), ("state", state)):
        _need(t, torch.float32, name)
    n = xbc.shape[0]
    inner = heads * head_dim
    if xbc.shape[1] != inner + 2 * groups * state_dim or dt.dtype != xbc.dtype or dt.stride(1) != 1 or tuple(dt.shape) != (n, heads):
        raise KernelError("ssm_scan: xbc or dt has the wrong shape")
    if tuple(state.shape[1:]) != (heads, head_dim, state_dim) or state_dim > 256:
        raise KernelError("ssm_scan: the state must be [slots, heads, head_dim, state_dim] with state_dim <= 256")
    y = torch.empty((n, inner), dtype=torch.float32, device=xbc.device)
    _check(ops_library().ss_ssm_scan(xbc.data_ptr(), xbc.shape[1], dt.data_ptr(), dt.stride(0), dt_bias.data_ptr(),
                                     a_log.data_ptr(), d_skip.data_ptr(), state.data_ptr(), y.data_ptr(),
                                     ctx.q_start.data_ptr(), ctx.seq_lens.data_ptr(), ctx.state_slots.data_ptr(),
                                     ctx.num_requests, heads, groups, head_dim, state_dim, state.shape[0], _code(xbc.dtype),
                                     error_word(xbc.device).data_ptr(), _stream(), int(not ctx.is_decode_only)), "ssm_scan")
    return y


def router(x: torch.Tensor, weight: torch.Tensor, top: int, renormalize: bool = False, *, softmax: bool = False,
           correction: torch.Tensor | None = None, groups: int = 1, keep: int = 1,
           extra: int = 0) -> "tuple[torch.Tensor, torch.Tensor] | tuple[torch.Tensor, torch.Tensor, torch.Tensor]":
    """Router: logits ``x @ weight.T`` in float32, scores their sigmoid (or, with ``softmax``, their softmax over all
    experts), the ``top`` largest per token chosen (the lower index on a tie).  ``correction`` (float32 [experts]) is
    added to the scores for the choice only.  ``groups`` > 1: the experts form that many equal groups of neighbours, a
    group's score is its largest choice score, and only experts of the ``keep`` best groups can be chosen.  Returns
    (int32 [N, top] experts, float32 [N, top] their scores without the correction, divided by their sum with
    ``renormalize``).  ``extra``: the last ``extra`` rows of ``weight`` are not experts; their logits ride along in the
    product and come back as a third result, float32 [N, extra]."""
    _need(x, None, "x")
    _need(weight, x.dtype, "router weight")
    n, hidden = x.shape
    experts = weight.shape[0] - int(extra)
    if (weight.shape[1] != hidden or not 1 <= top <= experts or experts > 1024 or extra < 0
            or (hidden + 3 + 2 * experts + groups) * 4 > 48 * 1024):
        raise KernelError("router: sizes out of range")
    if groups < 1 or experts % groups or not 1 <= keep <= groups or top > keep * (experts // groups):
        raise KernelError("router: the experts do not split into such groups, or too few are kept for the choices")
    if correction is not None:
        _need(correction, torch.float32, "correction")
        if correction.numel() != experts:
            raise KernelError("router: one correction per expert")
    ids = torch.empty((n, top), dtype=torch.int32, device=x.device)
    scores = torch.empty((n, top), dtype=torch.float32, device=x.device)
    rest = torch.empty((n, extra), dtype=torch.float32, device=x.device) if extra else None
    _check(ops_library().ss_router(x.data_ptr(), weight.data_ptr(), ids.data_ptr(), scores.data_ptr(), n, hidden, experts,
                                   int(top), int(renormalize), _code(x.dtype), _stream(), int(softmax), _ptr(correction),
                                   int(groups), int(keep), _ptr(rest), int(extra)), "router")
    return (ids, scores, rest) if extra else (ids, scores)


MOE_TILE = 64  # rows of one expert that a block of the grouped products takes


GROUPED_TCGEN05_ROWS = 1024  # from this many (token, choice) pairs the experts' products run the two-SM tcgen05 kernel


def moe_experts(x: torch.Tensor, ids: torch.Tensor, scores: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor,
                run: int | None = None) -> tuple[torch.Tensor, torch.Tensor | None]:
    """The chosen experts of every token: ``y[t, k] = W_down[e] (silu(W_gate[e] a) * (W_up[e] a))`` with
    ``e = ids[t, k]`` and ``a = scores[t, k] * x[t]`` (the score multiplies the expert's INPUT), rounded to the
    compute dtype.  ``gate_up`` [experts, 2 ff, hidden]: gate and up rows alternating in runs of ``run`` (default ff:
    all gate rows, then all up rows); ``down`` [experts, hidden, ff].

    Returns (terms, term_rows): either float32 [N, top, hidden] and None, or, from the tcgen05 path, bfloat16
    [N * top, hidden] in sorted order with int32 [N * top] saying where pair (t, k) stands (`group_norm` and
    `moe_combine` take both forms).  The same launches whatever the routing: the plan (pairs sorted by expert and cut
    into tiles), a gather of the scaled activations into sorted order, the up product with the activation, the down
    product.  bfloat16 with sizes in steps of 8 runs the products on the tensor cores: mma.sync tiles of 32 or 128
    sorted rows, or, with runs of 64 and many pairs, the grouped form of the two-SM tcgen05 kernel over tiles of 256;
    everything else runs them on CUDA cores."""
    n, hidden = x.shape
    experts, two_ff, _ = gate_up.shape
    ff, top = two_ff // 2, ids.shape[1]
    run = ff if run is None else int(run)
    _need(x, None, "x")
    _need(gate_up, x.dtype, "gate_up")
    _need(down, x.dtype, "down")
    _need(ids, torch.int32, "ids")
    _need(scores, torch.float32, "scores")
    if tuple(down.shape) != (experts, hidden, ff) or gate_up.shape[2] != hidden or run < 1 or ff % run:
        raise KernelError("moe_experts: weights of the wrong shape")
    a = n * top
    tensor_cores = x.dtype == torch.bfloat16 and hidden % 8 == 0 and ff % 8 == 0
    tcgen05 = tensor_cores and run == 64 and hidden % 16 == 0 and a >= GROUPED_TCGEN05_ROWS
    tile = MOE_TILE if not tensor_cores else (256 if tcgen05 else (128 if a >= 96 * experts else 32))
    max_tiles = (a + tile - 1) // tile + experts
    plan = torch.empty(2 * a + 3 * max_tiles, dtype=torch.int32, device=x.device)
    perm, place, tile_expert = plan[:a], plan[a: 2 * a], plan[2 * a: 2 * a + max_tiles]
    tile_row0, tile_rows = plan[2 * a + max_tiles: 2 * a + 2 * max_tiles], plan[2 * a + 2 * max_tiles:]
    lib = ops_library()
    _check(lib.ss_moe_plan(ids.data_ptr(), perm.data_ptr(), tile_expert.data_ptr(), tile_row0.data_ptr(),
                           tile_rows.data_ptr(), a, experts, tile, max_tiles, place.data_ptr(), _stream(), experts), "moe_plan")
    hidden_act = torch.empty((a, ff), dtype=x.dtype, device=x.device)
    lists = (perm.data_ptr(), tile_expert.data_ptr(), tile_row0.data_ptr(), tile_rows.data_ptr())
    if tensor_cores:
        gathered = torch.empty((a, hidden), dtype=x.dtype, device=x.device)
        _check(lib.ss_moe_gather(x.data_ptr(), scores.data_ptr(), perm.data_ptr(), gathered.data_ptr(), a, top, hidden,
                                 _stream()), "moe_gather")
    if tcgen05:
        err = error_word(x.device).data_ptr()
        y_sorted = torch.empty((a, hidden), dtype=x.dtype, device=x.device)
        _check(gemm_library().ss_gemm_tc5_grouped(gathered.data_ptr(), gate_up.data_ptr(), hidden_act.data_ptr(), a, two_ff,
                                                  hidden, experts, two_ff, ff, 1, *lists[1:], max_tiles, err, _stream()),
               "moe_up")
        _check(gemm_library().ss_gemm_tc5_grouped(hidden_act.data_ptr(), down.data_ptr(), y_sorted.data_ptr(), a, hidden, ff,
                                                  experts, hidden, hidden, 0, *lists[1:], max_tiles, err, _stream()),
               "moe_down")
        return y_sorted, place
    y = torch.empty((n, top, hidden), dtype=torch.float32, device=x.device)
    if tensor_cores:
        _check(lib.ss_moe_gemm_mma(gathered.data_ptr(), gate_up.data_ptr(), *lists, hidden_act.data_ptr(), None, hidden, ff,
                                   max_tiles, tile, 1, run, int(a <= 4), _stream()), "moe_up")
        _check(lib.ss_moe_gemm_mma(hidden_act.data_ptr(), down.data_ptr(), *lists, None, y.data_ptr(), ff, hidden,
                                   max_tiles, tile, 0, 0, int(a <= 4), _stream()), "moe_down")
        return y, None
    _check(lib.ss_moe_gemm(x.data_ptr(), scores.data_ptr(), gate_up.data_ptr(), *lists, hidden_act.data_ptr(), None, top,
                           hidden, ff, max_tiles, 1, _code(x.dtype), run, _stream(), 0), "moe_up")
    _check(lib.ss_moe_gemm(hidden_act.data_ptr(), None, down.data_ptr(), *lists, None, y.data_ptr(), top, ff, hidden,
                           max_tiles, 0, _code(x.dtype), 0, _stream(), 0), "moe_down")
    return y, None


def moe_combine(y: torch.Tensor, shared: torch.Tensor | None, out_dtype: torch.dtype,
                term_rows: torch.Tensor | None = None, top: int = 1) -> torch.Tensor:
    """``sum_k y[t, k] + shared[t]`` rounded to ``out_dtype``: the chosen experts' outputs in the order of the choices,
    then the shared expert's.  ``y``: either form that `moe_experts` returns (with ``term_rows``: the sorted
    bfloat16 rows, ``top`` choices a token)."""
    if term_rows is None:
        _need(y, torch.float32, "expert outputs")
        n, top, hidden = y.shape
    else:
        _need(y, torch.bfloat16, "sorted expert outputs")
        _need(term_rows, torch.int32, "term_rows")
        n, hidden = term_rows.numel() // top, y.shape[1]
    if shared is not None:
        _need(shared, out_dtype, "shared expert output")
    out = torch.empty((n, hidden), dtype=out_dtype, device=y.device)
    _check(ops_library().ss_moe_combine(y.data_ptr() if term_rows is None else None, _ptr(shared), out.data_ptr(), n, hidden,
                                        top, _code(out_dtype), _ptr(y) if term_rows is not None else None, _ptr(term_rows),
                                        _stream()), "moe_combine")
    return out


def norm_rope_cache(rows: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor | None, kv: torch.Tensor | None,
                    n_q: int, n_kv: int, head_dim: int, *, inv_freq: torch.Tensor | None = None, rotary_dim: int = 0,
                    value_inv_freq: torch.Tensor | None = None, value_rotary_dim: int = 0, interleaved: bool = False,
                    q_weight: torch.Tensor | None = None, k_weight: torch.Tensor | None = None, norm_dim: int = 0,
                    eps: float = 0.0, write_cache: bool = True) -> None:
    """For a layer's projected heads (``rows`` [N, >= (n_q + 2 n_kv) * head_dim]: queries, keys, values): an RMS norm
    of every query and key head over its first ``norm_dim`` elements with a weight shared by the heads (float32
    [norm_dim]) BEFORE the rotation; the rotation of the first ``rotary_dim`` elements of queries and keys by
    position * ``inv_freq``; the rotation of the first ``value_rotary_dim`` elements of every value head by position *
    ``value_inv_freq``; pairs (i, i + dims / 2) or, ``interleaved``, (2i, 2i + 1).  Queries change in place; keys
    and values go to their pages ``kv`` [pages, 2, n_kv, page_size, head_dim] at ``slots``."""
    _need(rows, None, "projected rows")
    _need(positions, torch.int32, "positions")
    n, width = rows.shape
    if width < (n_q + 2 * n_kv) * head_dim:
        raise KernelError("the projected rows are narrower than their heads")
    for t, dims, what in ((inv_freq, rotary_dim, "inv_freq"), (value_inv_freq, value_rotary_dim, "value_inv_freq")):
        if dims:
            _need(t, torch.float32, what)
            if dims % 2 or dims > head_dim or t.numel() != dims // 2:
                raise KernelError(f"{what} must hold dims / 2 values, dims even and at most head_dim")
    if norm_dim:
        _need(q_weight, torch.float32, "q norm weight")
        if n_kv:
            _need(k_weight, torch.float32, "k norm weight")
        if q_weight.numel() != norm_dim or (n_kv and k_weight.numel() != norm_dim) or norm_dim > head_dim:
            raise KernelError("query/key norm weights must hold norm_dim values")
    write = bool(write_cache and n_kv and kv is not None and slots is not None)
    pages, page_size = 0, 1
    if write:
        _need(kv, rows.dtype, "kv pages")
        _need(slots, torch.int32, "slots")
        if kv.dim() != 5 or kv.shape[1] != 2 or kv.shape[2] != n_kv or kv.shape[4] != head_dim:
            raise KernelError(f"kv pages have shape {tuple(kv.shape)}, expected [pages, 2, {n_kv}, page, {head_dim}]")
        pages, page_size = kv.shape[0], kv.shape[3]
    _check(ops_library().ss_norm_rope_cache(rows.data_ptr(), width, positions.data_ptr(), _ptr(slots) if write else None,
                                            _ptr(inv_freq) if rotary_dim else None,
                                            _ptr(value_inv_freq) if value_rotary_dim else None,
                                            _ptr(q_weight) if norm_dim else None, _ptr(k_weight) if norm_dim and n_kv else None,
                                            _ptr(kv) if write else None, n, n_q, n_kv, head_dim, int(rotary_dim),
                                            int(value_rotary_dim), int(interleaved), int(norm_dim), float(eps), page_size,
                                            pages, _code(rows.dtype), error_word(rows.device).data_ptr(), _stream()),
           "norm_rope_cache")


def turn_heads(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, heads: int, head_dim: int, dims: int,
               interleaved: bool = False, sign: float = -1.0) -> None:
    """Rotate the first ``dims`` elements of every head of ``x`` [N, heads * head_dim] in place by
    ``sign * position * inv_freq`` (pairs as in `norm_rope_cache`): with ``sign`` -1 the turn back of heads' outputs
    that were summed over rotated values."""
    _need(x, None, "heads")
    _need(positions, torch.int32, "positions")
    _need(inv_freq, torch.float32, "inv_freq")
    if x.shape[1] != heads * head_dim or dims % 2 or dims > head_dim or inv_freq.numel() != dims // 2:
        raise KernelError("turn_heads: sizes do not match")
    _check(ops_library().ss_turn_heads(x.data_ptr(), positions.data_ptr(), inv_freq.data_ptr(), x.shape[0], heads, head_dim,
                                       int(dims), int(interleaved), float(sign), _code(x.dtype), _stream()), "turn_heads")


def soft_cap(x: torch.Tensor, cap: float | None, scale: float = 1.0) -> torch.Tensor:
    """``x <- cap * tanh(scale * x / cap)`` in place (float32); without a cap ``x <- scale * x``."""
    _need(x, torch.float32, "x")
    _check(ops_library().ss_soft_cap(x.data_ptr(), x.numel(), float(cap or 0.0), _stream(), float(scale)), "soft_cap")
    return x


# --------------------------------------------------------------------------- recurrent cells, latent attention

def embed_sum(token_ids: torch.Tensor, table: torch.Tensor, ctx, *, pair_table: torch.Tensor | None = None,
              pair_hash: tuple[int, int, int] | None = None, last_token: torch.Tensor | None = None,
              position_table: torch.Tensor | None = None, scale: float = 1.0, copies: int = 1) -> torch.Tensor:
    """An embedding that is a sum of rows, float32 [N, hidden] (``copies`` > 1: [N, copies, hidden], every copy alike):
    ``scale * table[token]``, plus ``pair_table[(previous * mul_prev + token * mul_cur) mod buckets]`` with
    ``pair_hash`` = (buckets, mul_prev, mul_cur) and row ``buckets`` for a request's first token, plus
    ``position_table[position]``.  The token in front of a step's first row is the request's state ``last_token``
    (int32 [slots]), which the kernel leaves holding the step's last token."""
    _need(token_ids, torch.int32, "token_ids")
    _need(table, None, "embedding table")
    n, (vocab, hidden) = token_ids.numel(), table.shape
    buckets = mul_prev = mul_cur = 0
    if pair_table is not None:
        _need(pair_table, table.dtype, "pair table")
        _need(last_token, torch.int32, "last_token")
        buckets, mul_prev, mul_cur = (int(v) for v in pair_hash)
        if buckets < 1 or tuple(pair_table.shape) != (buckets + 1, hidden):
            raise KernelError("the pair table must be [buckets + 1, hidden]")
    if position_table is not None:
        _need(position_table, table.dtype, "position table")
        if position_table.shape[1] != hidden:
            raise KernelError("the position table must be [positions, hidden]")
    out = torch.empty((n, hidden) if copies == 1 else (n, copies, hidden), dtype=torch.float32, device=table.device)
    _check(ops_library().ss_embed_sum(token_ids.data_ptr(), ctx.positions.data_ptr(), table.data_ptr(), _ptr(pair_table),
                                      _ptr(position_table), out.data_ptr(), _ptr(last_token), ctx.q_start.data_ptr(),
                                      ctx.seq_lens.data_ptr(), ctx.state_slots.data_ptr(), ctx.num_requests, n, hidden, vocab,
                                      int(copies), buckets, mul_prev, mul_cur,
                                      position_table.shape[0] if position_table is not None else 0,
                                      last_token.shape[0] if last_token is not None else 0, float(scale), _code(table.dtype),
                                      error_word(table.device).data_ptr(), _stream()), "embed_sum")
    return out


def matrix_cell(qkv: torch.Tensor, gates: torch.Tensor, bias_i: torch.Tensor | None, bias_f: torch.Tensor | None, cap: float,
                q_scale: float, memory: torch.Tensor, peak: torch.Tensor, ctx, heads: int, dim: int, vdim: int
                ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """The matrix-memory recurrence over each request's tokens, continued from and left in ``memory`` (float32
    [slots, heads, vdim + 1, dim]: S column by column, the last column the normaliser n) and ``peak`` (float32
    [slots, heads], the running maximum m, which starts at 0).  A row of ``qkv`` starts with [q: heads * dim |
    k: heads * dim | v: heads * vdim]; ``gates`` float32 [N, >= 2 heads] holds the raw input and forget gates.  With
    ``i = cap tanh((a + bias_i) / cap)`` and ``f = logsigmoid(cap tanh((b + bias_f) / cap))``:
    ``m' = max(f + m, i)``, ``S <- exp(f + m - m') S + exp(i - m') k v^T``, n likewise with k alone.
    Returns (``S^T (q_scale q)`` float32 [N, heads * vdim], ``n . (q_scale q)`` [N, heads], m [N, heads])."""
    _need(qkv, None, "q, k and v")
    _need(gates, torch.float32, "gates")
    _need(memory, torch.float32, "memory")
    _need(peak, torch.float32, "peak")
    n = qkv.shape[0]
    if qkv.shape[1] < heads * (2 * dim + vdim) or gates.shape[0] != n or gates.shape[1] < 2 * heads:
        raise KernelError("matrix_cell: q, k, v or the gates have the wrong shape")
    if tuple(memory.shape[1:]) != (heads, vdim + 1, dim) or tuple(peak.shape[1:]) != (heads,) or not 1 <= dim <= 256:
        raise KernelError("matrix_cell: the memory must be [slots, heads, vdim + 1, dim] with dim <= 256, the peak [slots, heads]")
    for b in (bias_i, bias_f):
        if b is not None:
            _need(b, torch.float32, "gate bias")
    num = torch.empty((n, heads * vdim), dtype=torch.float32, device=qkv.device)
    nq = torch.empty((n, heads), dtype=torch.float32, device=qkv.device)
    peaks = torch.empty((n, heads), dtype=torch.float32, device=qkv.device)
    _check(ops_library().ss_matrix_cell(qkv.data_ptr(), qkv.stride(0), gates.data_ptr(), gates.stride(0), _ptr(bias_i),
                                        _ptr(bias_f), float(cap), float(q_scale), memory.data_ptr(), peak.data_ptr(),
                                        num.data_ptr(), nq.data_ptr(), peaks.data_ptr(), ctx.q_start.data_ptr(),
                                        ctx.seq_lens.data_ptr(), ctx.state_slots.data_ptr(), ctx.num_requests, heads, dim, vdim,
                                        memory.shape[0], _code(qkv.dtype), error_word(qkv.device).data_ptr(), _stream()),
           "matrix_cell")
    return num, nq, peaks


def cell_output(num: torch.Tensor, nq: torch.Tensor, peaks: torch.Tensor, weight: torch.Tensor, gate: torch.Tensor,
                heads: int, vdim: int, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """The matrix-memory cell's output: ``o = num / (max(|nq|, exp(-m)) + 1e-6)``, every head of ``o`` divided by its root
    mean square (``eps`` inside the root), times ``weight`` (float32 [heads * vdim]), times ``sigmoid(gate)`` (a view
    [N, heads * vdim] in ``out_dtype`` with unit inner stride).  Returns [N, heads * vdim] in ``out_dtype``."""
    for name, t in (("num", num), ("nq", nq), ("peaks", peaks), ("weight", weight)):
        _need(t, torch.float32, name)
    n = num.shape[0]
    if gate.dtype != out_dtype or gate.stride(1) != 1 or tuple(gate.shape) != (n, heads * vdim) or weight.numel() != heads * vdim:
        raise KernelError("cell_output: the gate or the weight has the wrong shape")
    out = torch.empty((n, heads * vdim), dtype=out_dtype, device=num.device)
    _check(ops_library().ss_cell_output(num.data_ptr(), nq.data_ptr(), peaks.data_ptr(), weight.data_ptr(), gate.data_ptr(),
                                        gate.stride(0), out.data_ptr(), n, heads, vdim, float(eps), _code(out_dtype),
                                        _stream()), "cell_output")
    return out


def gated_recurrence(proj: torch.Tensor, width: int, state: torch.Tensor, ctx, bias: torch.Tensor | None = None,
                     portions: bool | None = None) -> torch.Tensor:
    """A gated recurrence per channel over each request's tokens, continued from and left in ``state`` (float32
    [slots, width]).  A row of ``proj`` is [z | u | g], ``width`` each; ``bias`` (float32 [2 width]) is added to z and u
    in float32.  ``z' = sigmoid(z)``; the candidate is ``u + 1/2`` where ``u >= 0`` and ``sigmoid(u)`` below;
    ``S <- (1 - z') S + z' candidate``; returns ``S silu(g)`` [N, width] in the dtype of ``proj``.

    ``portions`` (default: every step that is not decode-only) runs the kernel that also cuts a request's tokens into
    segments: a segment acts on the state in front of it as ``S -> A S + B``, the segments' (A, B) are chained in order,
    and each segment is then walked from its own starting state.  Otherwise a thread walks all rows of a channel."""
    if portions is None:
        portions = not ctx.is_decode_only
    _need(proj, None, "projection")
    _need(state, torch.float32, "state")
    if bias is not None:
        _need(bias, torch.float32, "gate biases")
        if bias.numel() != 2 * width:
            raise KernelError("gated_recurrence: the biases must hold 2 * width values")
    if proj.shape[1] < 3 * width or tuple(state.shape[1:]) != (width,):
        raise KernelError("gated_recurrence: the projection or the state has the wrong shape")
    out = torch.empty((proj.shape[0], width), dtype=proj.dtype, device=proj.device)
    _check(ops_library().ss_gated_recurrence(proj.data_ptr(), proj.stride(0), _ptr(bias), state.data_ptr(), out.data_ptr(),
                                             ctx.q_start.data_ptr(), ctx.seq_lens.data_ptr(), ctx.state_slots.data_ptr(),
                                             ctx.num_requests, width, state.shape[0], _code(proj.dtype),
                                             error_word(proj.device).data_ptr(), _stream(), int(bool(portions))),
           "gated_recurrence")
    return out


def xielu(x: torch.Tensor, a: float, b: float) -> torch.Tensor:
    """In place: ``a x^2 + x / 2`` where ``x > 0``, ``b (exp(x) - 1 - x) + x / 2`` elsewhere."""
    _need(x, None, "x")
    _check(ops_library().ss_xielu(x.data_ptr(), x.data_ptr(), x.numel(), float(a), float(b), _code(x.dtype), _stream()), "xielu")
    return x


def latent_rows(down: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor | None, kv: torch.Tensor | None,
                q_weight: torch.Tensor, kv_weight: torch.Tensor | None, inv_freq: torch.Tensor | None, mscale: float,
                q_rank: int, kv_rank: int, rot_dim: int, eps: float) -> torch.Tensor:
    """The latents of a latent-attention layer.  A row of ``down`` is [query latent: q_rank | key/value latent: kv_rank |
    shared key part: rot_dim | ...].  Returns ``rmsnorm(query latent) * q_weight`` [N, q_rank]; with ``kv_rank`` > 0 the
    key/value latent is normed likewise (``kv_weight``), the shared key part rotated by the row's position (pairs
    (i, i + rot_dim / 2), angle ``position * inv_freq[i]``, cosines and sines times ``mscale``; ``inv_freq`` None: not
    rotated), and the pages ``kv`` [pages, 2, 1, page_size, D] take the key row [rotated part | latent | zeros] and the
    value row [latent | zeros] at ``slots``."""
    _need(down, None, "down projection")
    _need(positions, torch.int32, "positions")
    _need(q_weight, torch.float32, "query latent's norm weight")
    n = down.shape[0]
    dp = page_size = pages = 0
    if kv_rank > 0:
        _need(kv, down.dtype, "kv pages")
        _need(slots, torch.int32, "slots")
        _need(kv_weight, torch.float32, "latent's norm weight")
        if kv.dim() != 5 or kv.shape[1] != 2 or kv.shape[2] != 1 or kv.shape[4] < kv_rank + rot_dim:
            raise KernelError("latent_rows: the pages must be [pages, 2, 1, page_size, D] with D >= kv_rank + rot_dim")
        pages, page_size, dp = kv.shape[0], kv.shape[3], kv.shape[4]
    if inv_freq is not None:
        _need(inv_freq, torch.float32, "inv_freq")
        if inv_freq.numel() != rot_dim // 2:
            raise KernelError("inv_freq must hold rot_dim / 2 values")
    if down.shape[1] < q_rank + (kv_rank + rot_dim if kv_rank > 0 else 0) or rot_dim % 2:
        raise KernelError("latent_rows: the down projection is narrower than its parts, or rot_dim is odd")
    cq = torch.empty((n, q_rank), dtype=down.dtype, device=down.device)
    _check(ops_library().ss_latent_rows(down.data_ptr(), down.stride(0), positions.data_ptr(), _ptr(slots) if kv_rank > 0 else None,
                                        q_weight.data_ptr(), _ptr(kv_weight), _ptr(inv_freq), float(mscale), cq.data_ptr(),
                                        _ptr(kv) if kv_rank > 0 else None, n, q_rank, kv_rank, rot_dim, dp, page_size, pages,
                                        float(eps), _code(down.dtype), error_word(down.device).data_ptr(), _stream()),
           "latent_rows")
    return cq


HEAD_PRODUCT_LIBRARY_ROWS = 128  # rows from which the per-head products go to the library's batched product


def head_product(x: torch.Tensor, x_head: int, weight: torch.Tensor, out: torch.Tensor, out_head: int, *, turn: int = 0,
                 pad_to: int | None = None, positions: torch.Tensor | None = None, inv_freq: torch.Tensor | None = None,
                 mscale: float = 1.0, gates: torch.Tensor | None = None) -> torch.Tensor:
    """A product per head: ``out[n, h, turn + o] = f * sum_i x[n, h, i] * weight[h, i, o]`` with ``weight`` [H, I, O], head h
    of a row of ``x`` starting at column ``h * x_head`` and of ``out`` at ``h * out_head``; float32 accumulation in the
    order of i.  ``turn`` > 0: the ``turn`` elements of x behind the I inputs are rotated by the row's position (pairs
    (i, i + turn / 2), ``inv_freq`` None: copied) into ``out[n, h, :turn]``.  Columns from ``turn + O`` to ``pad_to`` are
    zeroed.  ``gates`` (a view [N, H] in the dtype of x, unit inner stride): ``f = sigmoid(gates[n, h])``, else 1.

    bfloat16 with at least ``HEAD_PRODUCT_LIBRARY_ROWS`` rows (prompt portions): the products are one batched library
    matrix product over strided views of ``x`` and ``out`` (as `linear` falls to the library product), and this
    package's kernel then only rotates, zeroes the padding and applies ``f`` in place."""
    _need(x, None, "x")
    _need(weight, x.dtype, "weights per head")
    _need(out, x.dtype, "output")
    h, i, o = weight.shape
    n = x.shape[0]
    pad_to = turn + o if pad_to is None else int(pad_to)
    if x.shape[1] < (h - 1) * x_head + i + turn or out.shape[1] < (h - 1) * out_head + pad_to or out.shape[0] != n:
        raise KernelError("head_product: x or out is narrower than its heads")
    if turn:
        _need(positions, torch.int32, "positions")
    gate_stride = scale_col = 0
    gate_ptr = None
    if gates is not None:
        if gates.dtype != x.dtype or gates.stride(1) != 1 or tuple(gates.shape) != (n, h):
            raise KernelError("head_product: gates must be a view [N, H] in the dtype of x")
        gate_ptr, gate_stride = gates.data_ptr(), gates.stride(0)
    else:
        scale_col = -1
    weight_ptr = weight.data_ptr()
    if x.dtype == torch.bfloat16 and n >= HEAD_PRODUCT_LIBRARY_ROWS:
        torch.bmm(x.as_strided((h, n, i), (int(x_head), x.stride(0), 1)), weight,
                  out=out.as_strided((h, n, o), (int(out_head), out.stride(0), 1), out.storage_offset() + int(turn)))
        if not turn and pad_to == o and gates is None:
            return out
        weight_ptr = None
    _check(ops_library().ss_head_product(x.data_ptr(), x.stride(0), int(x_head), weight_ptr, out.data_ptr(),
                                         out.stride(0), int(out_head), n, h, i, o, int(turn), pad_to, _ptr(positions),
                                         _ptr(inv_freq), float(mscale), gate_ptr, gate_stride, scale_col, _code(x.dtype),
                                         _stream()), "head_product")
    return out



# --------------------------------------------------------------------------- decayed linear attention, gated linear recurrence

def decay_attention(proj: torch.Tensor, decay: torch.Tensor, state: torch.Tensor, ctx, heads: int, dim: int,
                    value_dim: int) -> torch.Tensor:
    """Linear attention with a fixed decay per head over each request's tokens, continued from and left in ``state``
    (float32 [slots, heads, dim, value_dim]).  A row of ``proj`` starts with the heads' queries, then keys (``dim``
    each), then values (``value_dim``), all before their activation; whatever follows is left alone.  Per head h, token
    by token: ``S <- decay[h] S + silu(k) silu(v)^T``, ``o = S^T silu(q)``.  Returns o float32 [N, heads * value_dim]."""
    _need(proj, None, "projected rows")
    _need(decay, torch.float32, "decay")
    _need(state, torch.float32, "state")
    n = proj.shape[0]
    if proj.shape[1] < heads * (2 * dim + value_dim) or decay.numel() != heads or not 1 <= dim <= 256:
        raise KernelError("decay_attention: the rows are narrower than their heads, or sizes out of range")
    if tuple(state.shape[1:]) != (heads, dim, value_dim):
        raise KernelError("decay_attention: the state must be [slots, heads, dim, value_dim]")
    out = torch.empty((n, heads * value_dim), dtype=torch.float32, device=proj.device)
    _check(ops_library().ss_decay_attention(proj.data_ptr(), proj.stride(0), decay.data_ptr(), state.data_ptr(),
                                            out.data_ptr(), ctx.q_start.data_ptr(), ctx.seq_lens.data_ptr(),
                                            ctx.state_slots.data_ptr(), ctx.num_requests, heads, dim, value_dim,
                                            state.shape[0], _code(proj.dtype), error_word(proj.device).data_ptr(), _stream()),
           "decay_attention")
    return out


def gated_rmsnorm(x: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps) * weight * sigmoid(gate)`` row by row: ``x`` float32 [N, C], ``gate`` a view [N, C] in
    ``out_dtype`` with unit inner stride, ``weight`` float32 [C]; float32 arithmetic, one rounding."""
    _need(x, torch.float32, "x")
    _need(weight, torch.float32, "norm weight")
    n, c = x.shape
    if gate.dtype != out_dtype or tuple(gate.shape) != (n, c) or gate.stride(1) != 1 or weight.numel() != c:
        raise KernelError("gated_rmsnorm: the gate must be [N, C] in the compute dtype with unit inner stride, the weight [C]")
    out = torch.empty((n, c), dtype=out_dtype, device=x.device)
    _check(ops_library().ss_gated_rmsnorm(x.data_ptr(), gate.data_ptr(), gate.stride(0), weight.data_ptr(), out.data_ptr(),
                                          n, c, float(eps), _code(out_dtype), _stream()), "gated_rmsnorm")
    return out


BLOCK_GATES_LIBRARY_ROWS = 128  # rows from which the gates' block products go to the library's batched product


def block_gates(u: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Two gates' pre-activations from square blocks of the input: ``u`` [N, blocks * bs]; ``weight`` [blocks, 2 bs, bs]
    (per block the first gate's rows, then the second's).  Returns float32 [blocks, N, 2 bs]:
    ``pre[b, t] = weight[b] @ u[t, b bs : (b + 1) bs]``, accumulated in float32.  Many bfloat16 rows run the library's
    batched product with a float32 result (its inputs are the same bfloat16 numbers, its sums float32)."""
    _need(u, None, "u")
    _need(weight, u.dtype, "gate weights")
    n = u.shape[0]
    blocks, two_bs, bs = weight.shape
    if two_bs != 2 * bs or u.shape[1] != blocks * bs:
        raise KernelError("block_gates: weight must be [blocks, 2 bs, bs] and u [N, blocks * bs]")
    if u.dtype == torch.bfloat16 and n >= BLOCK_GATES_LIBRARY_ROWS and bs % 8 == 0:
        return torch.bmm(u.view(n, blocks, bs).transpose(0, 1), weight.transpose(1, 2), out_dtype=torch.float32)
    pre = torch.empty((blocks, n, two_bs), dtype=torch.float32, device=u.device)
    _check(ops_library().ss_block_gates(u.data_ptr(), u.stride(0), weight.data_ptr(), None, pre.data_ptr(), n, blocks, bs,
                                        _code(u.dtype), _stream()), "block_gates")
    return pre


RECURRENCE_SEGMENTS = 16  # warps that share a request's rows of a step with prompt portions


def gated_linear_recurrence(pre: torch.Tensor, bias: torch.Tensor | None, u: torch.Tensor, y: torch.Tensor, lam: torch.Tensor,
                            rate: float, state: torch.Tensor, ctx) -> torch.Tensor:
    """The real-gated linear recurrence over each request's tokens, continued from and left in ``state`` (float32
    [slots, C]).  ``pre`` float32 [blocks, N, 2 bs] (`block_gates`), ``bias`` float32 [blocks, 2 bs] or None, ``u``
    [N, C] the recurrence's input, ``y`` a view [N, C] (unit inner stride) of the other branch before its activation,
    ``lam`` float32 [C].  Per channel: ``r = sigmoid(pre1 + bias1)``, ``i = sigmoid(pre2 + bias2)``,
    ``a = exp(-rate r softplus(lam))``, ``S <- a S + sqrt(1 - a^2) i u``; returns ``S gelu_tanh(y)`` [N, C] in the
    dtype of ``u``.  In steps with prompt portions a request's rows are cut into `RECURRENCE_SEGMENTS` segments that
    are walked side by side (``pre`` is used as scratch and holds other values afterwards)."""
    _need(pre, torch.float32, "gate pre-activations")
    _need(u, None, "u")
    _need(lam, torch.float32, "lam")
    _need(state, torch.float32, "state")
    blocks, n, two_bs = pre.shape
    bs, c = two_bs // 2, u.shape[1]
    if u.shape[0] != n or blocks * bs != c or lam.numel() != c or tuple(state.shape[1:]) != (c,):
        raise KernelError("gated_linear_recurrence: shapes do not match")
    if y.dtype != u.dtype or tuple(y.shape) != (n, c) or y.stride(1) != 1:
        raise KernelError("gated_linear_recurrence: y must be a view [N, C] with unit inner stride in the dtype of u")
    if bias is not None:
        _need(bias, torch.float32, "gate biases")
        if bias.numel() != blocks * two_bs:
            raise KernelError("gated_linear_recurrence: one bias per gate and channel")
    out = torch.empty((n, c), dtype=u.dtype, device=u.device)
    _check(ops_library().ss_gated_linear_recurrence(pre.data_ptr(), _ptr(bias), u.data_ptr(), y.data_ptr(), y.stride(0),
                                                    lam.data_ptr(), float(rate), state.data_ptr(), out.data_ptr(),
                                                    ctx.q_start.data_ptr(), ctx.seq_lens.data_ptr(), ctx.state_slots.data_ptr(),
                                                    ctx.num_requests, n, c, bs, state.shape[0], _code(u.dtype),
                                                    error_word(u.device).data_ptr(), _stream(),
                                                    1 if ctx.is_decode_only else RECURRENCE_SEGMENTS), "gated_linear_recurrence")
    return out


def head_gate(x: torch.Tensor, gate: torch.Tensor, heads: int, head_dim: int) -> None:
    """``x[t, h * D + d] *= sigmoid(gate[t, h])`` in place: ``x`` [N, heads * D] contiguous, ``gate`` a view [N, heads]
    with unit inner stride in the same dtype."""
    _need(x, None, "x")
    n = x.shape[0]
    if x.shape[1] != heads * head_dim or gate.dtype != x.dtype or tuple(gate.shape) != (n, heads) or gate.stride(1) != 1:
        raise KernelError("head_gate: x must be [N, heads * D] and the gate a view [N, heads] of the same dtype")
    _check(ops_library().ss_head_gate(x.data_ptr(), gate.data_ptr(), gate.stride(0), n, heads, head_dim, _code(x.dtype),
                                      _stream()), "head_gate")


def scaled_sum(a: torch.Tensor, scale_a: float, b: torch.Tensor, scale_b: float) -> torch.Tensor:
    """``scale_a * a + scale_b * b`` element by element, formed in float32 and rounded once."""
    _need(a, None, "a")
    _need(b, a.dtype, "b")
    if a.shape != b.shape:
        raise KernelError("scaled_sum: shapes differ")
    out = torch.empty_like(a)
    _check(ops_library().ss_scaled_sum(a.data_ptr(), float(scale_a), b.data_ptr(), float(scale_b), out.data_ptr(), a.numel(),
                                       _code(a.dtype), _stream()), "scaled_sum")
    return out


def relu_square(x: torch.Tensor, cols: int | None = None) -> torch.Tensor:
    """``relu(x)^2`` of the first ``cols`` columns (default: all) of ``x`` [N, width] as a new contiguous [N, cols]."""
    if x.dim() != 2 or x.stride(1) != 1 or not x.is_cuda:
        raise KernelError("relu_square takes a CUDA tensor [N, width] with unit inner stride")
    cols = x.shape[1] if cols is None else int(cols)
    out = torch.empty((x.shape[0], cols), dtype=x.dtype, device=x.device)
    _check(ops_library().ss_relu_square(x.data_ptr(), x.stride(0), out.data_ptr(), x.shape[0], cols, _code(x.dtype),
                                        _stream()), "relu_square")
    return out


def moe_experts_single(x: torch.Tensor, ids: torch.Tensor, up: torch.Tensor, down: torch.Tensor,
                       slots: int | None = None) -> tuple[torch.Tensor, torch.Tensor | None]:
    """The chosen experts of every token for experts without a gate branch: ``y[t, k] = W_down[e] relu(W_up[e] x[t])^2``
    with ``e = ids[t, k]``; no weight is applied here (`moe_mix` weighs the outputs).  ``up`` [experts, ff, hidden],
    ``down`` [experts, hidden, ff].  ``slots`` (default: experts): ids from ``experts`` up to ``slots`` name experts
    without weights; their terms are not computed (and must not be read).  Returns what `moe_experts` returns, by the
    same three routes (CUDA cores; mma.sync tiles; the grouped two-SM tcgen05 kernel with the activation behind it)."""
    n, hidden = x.shape
    experts, ff, _ = up.shape
    top = ids.shape[1]
    slots = experts if slots is None else int(slots)
    _need(x, None, "x")
    _need(up, x.dtype, "up")
    _need(down, x.dtype, "down")
    _need(ids, torch.int32, "ids")
    if tuple(down.shape) != (experts, hidden, ff) or up.shape[2] != hidden or slots < experts or slots > 1024:
        raise KernelError("moe_experts_single: weights of the wrong shape")
    a = n * top
    tensor_cores = x.dtype == torch.bfloat16 and hidden % 8 == 0 and ff % 8 == 0
    tcgen05 = tensor_cores and hidden % 16 == 0 and ff % 16 == 0 and a >= GROUPED_TCGEN05_ROWS
    tile = MOE_TILE if not tensor_cores else (256 if tcgen05 else (128 if a >= 96 * experts else 32))
    max_tiles = (a + tile - 1) // tile + slots
    plan = torch.empty(2 * a + 3 * max_tiles, dtype=torch.int32, device=x.device)
    perm, place, tile_expert = plan[:a], plan[a: 2 * a], plan[2 * a: 2 * a + max_tiles]
    tile_row0, tile_rows = plan[2 * a + max_tiles: 2 * a + 2 * max_tiles], plan[2 * a + 2 * max_tiles:]
    lib = ops_library()
    _check(lib.ss_moe_plan(ids.data_ptr(), perm.data_ptr(), tile_expert.data_ptr(), tile_row0.data_ptr(),
                           tile_rows.data_ptr(), a, slots, tile, max_tiles, place.data_ptr(), _stream(), experts), "moe_plan")
    hidden_act = torch.empty((a, ff), dtype=x.dtype, device=x.device)
    lists = (perm.data_ptr(), tile_expert.data_ptr(), tile_row0.data_ptr(), tile_rows.data_ptr())
    if tensor_cores:
        gathered = torch.empty((a, hidden), dtype=x.dtype, device=x.device)
        _check(lib.ss_moe_gather(x.data_ptr(), None, perm.data_ptr(), gathered.data_ptr(), a, top, hidden, _stream()),
               "moe_gather")
    if tcgen05:
        err = error_word(x.device).data_ptr()
        y_sorted = torch.empty((a, hidden), dtype=x.dtype, device=x.device)
        _check(gemm_library().ss_gemm_tc5_grouped(gathered.data_ptr(), up.data_ptr(), hidden_act.data_ptr(), a, ff, hidden,
                                                  experts, ff, ff, 0, *lists[1:], max_tiles, err, _stream()), "moe_up")
        _check(lib.ss_relu_square(hidden_act.data_ptr(), ff, hidden_act.data_ptr(), a, ff, _code(x.dtype), _stream()),
               "relu_square")
        _check(gemm_library().ss_gemm_tc5_grouped(hidden_act.data_ptr(), down.data_ptr(), y_sorted.data_ptr(), a, hidden, ff,
                                                  experts, hidden, hidden, 0, *lists[1:], max_tiles, err, _stream()),
               "moe_down")
        return y_sorted, place
    y = torch.empty((n, top, hidden), dtype=torch.float32, device=x.device)
    if tensor_cores:
        _check(lib.ss_moe_gemm_mma(gathered.data_ptr(), up.data_ptr(), *lists, hidden_act.data_ptr(), None, hidden, ff,
                                   max_tiles, tile, 0, 0, int(a <= 4), _stream()), "moe_up")
        _check(lib.ss_moe_gemm_mma(hidden_act.data_ptr(), down.data_ptr(), *lists, None, y.data_ptr(), ff, hidden,
                                   max_tiles, tile, 0, 0, int(a <= 4), _stream()), "moe_down")
        return y, None
    _check(lib.ss_moe_gemm(x.data_ptr(), None, up.data_ptr(), *lists, hidden_act.data_ptr(), None, top, hidden, ff,
                           max_tiles, 0, _code(x.dtype), 0, _stream(), 1), "moe_up")
    _check(lib.ss_moe_gemm(hidden_act.data_ptr(), None, down.data_ptr(), *lists, None, y.data_ptr(), top, ff, hidden,
                           max_tiles, 0, _code(x.dtype), 0, _stream(), 0), "moe_down")
    return y, None


def moe_mix(y: torch.Tensor, term_rows: torch.Tensor | None, ids: torch.Tensor, weights: torch.Tensor | None, experts: int,
            x: torch.Tensor, shared: torch.Tensor | None = None, shared_gate: torch.Tensor | None = None) -> torch.Tensor:
    """``sum_k weights[t, k] * term(t, k) + sigmoid(shared_gate[t]) * shared[t]`` in float32, in the order of the
    choices, rounded once to the dtype of ``x``.  ``term(t, k)`` is expert ``ids[t, k]``'s output in either form that
    `moe_experts` returns, or, for an id from ``experts`` on (an expert that hands its input on), ``x[t]``.
    ``weights`` None: ones; ``shared_gate`` (float32, one logit per token, any stride) None: the shared expert's
    output as it is."""
    _need(x, None, "x")
    _need(ids, torch.int32, "ids")
    n, hidden = x.shape
    top = ids.shape[1]
    if term_rows is None:
        _need(y, torch.float32, "expert outputs")
        if tuple(y.shape) != (n, top, hidden):
            raise KernelError("moe_mix: the experts' outputs must be [N, top, hidden]")
    else:
        _need(y, torch.bfloat16, "sorted expert outputs")
        _need(term_rows, torch.int32, "term_rows")
        if x.dtype != torch.bfloat16 or y.shape[1] != hidden or term_rows.numel() != n * top:
            raise KernelError("moe_mix: sorted rows come with bfloat16 inputs and one place per choice")
    if weights is not None:
        _need(weights, torch.float32, "weights")
    if shared is not None:
        _need(shared, x.dtype, "shared expert output")
    gate_stride = 0
    if shared_gate is not None:
        if shared is None or shared_gate.dtype != torch.float32 or shared_gate.shape[0] != n:
            raise KernelError("moe_mix: the shared expert's gate is one float32 logit per token")
        gate_stride = shared_gate.stride(0)
    out = torch.empty((n, hidden), dtype=x.dtype, device=x.device)
    _check(ops_library().ss_moe_mix(y.data_ptr() if term_rows is None else None, _ptr(y) if term_rows is not None else None,
                                    _ptr(term_rows), ids.data_ptr(), _ptr(weights), int(experts), x.data_ptr(), _ptr(shared),
                                    _ptr(shared_gate), gate_stride, out.data_ptr(), n, hidden, top, _code(x.dtype), _stream()),
           "moe_mix")
    return out


def set_programmatic_launch(enabled: bool) -> None:
    """Turn programmatic dependent launch of this package's kernels on or off (on by default)."""
    libs = [ops_library(), gemm_library()] + [lib for key, lib in _state.items() if isinstance(key, str) and key.startswith("attn")]
    for lib in libs:
        lib.ss_set_pdl.argtypes = [c_int]
        lib.ss_set_pdl.restype = None
        lib.ss_set_pdl(int(enabled))
    _state["pdl"] = bool(enabled)


__all__ = ["KernelError", "KernelBuildError", "embedding", "add_rmsnorm", "hc_norm", "linear_hc_rmsnorm", "rope_norm_cache", "glu_limited", "gate_up_glu", "sigmoid_gate", "key_span", "rope_and_cache", "swiglu",
           "gemm_simt", "paged_attention_simt", "paged_attention", "fuses_rope", "paged_attention_prefill", "paged_attention_prefill_tcgen05", "prefill_key_parts", "tcgen05_attention_fits", "tcgen05_prefill_fits", "paged_attention_decode", "decode_scratch", "decode_slices", "is_long_context", "require_cuda", "argmax", "sample", "mark_seen", "gather_tokens", "prepare_decode", "gemm_tcgen05", "gemm_tcgen05_many", "many_tokens_fits", "many_tokens_swiglu_fits", "gemm_plan", "gemm_library", "gate_up_swiglu", "set_programmatic_launch", "launch_count", "count_launches", "sm_count", "linear", "linear_add_rmsnorm", "adds_to_stream", "takes_pending_norm", "PendingNorm", "set_norm_fusion", "check_errors", "raise_for_status", "error_word", "ops_library",
           "attention_library", "group_norm", "round_stream", "conv_silu", "ssm_scan", "router", "moe_experts", "moe_combine",
           "norm_rope_cache", "turn_heads", "soft_cap", "embed_sum", "matrix_cell", "cell_output", "gated_recurrence", "xielu",
           "latent_rows", "head_product", "decay_attention", "gated_rmsnorm", "block_gates", "gated_linear_recurrence", "head_gate",
           "scaled_sum", "relu_square", "moe_experts_single", "moe_mix"]
