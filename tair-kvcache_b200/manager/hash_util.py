"""Batched chained block hash on the GPU.

GenKeyVectorBatch is GenKeyVector (kv_cache_manager/manager/cache_manager.cc:76-87) for many
requests in one launch; ApplyPrefixHashBatch is ApplyPrefixHash
(kv_cache_manager/optimizer/trace_converter/trace_util.cc:47-56), i.e. block size 1.
"""
import ctypes

import numpy as np
import torch

from .. import _cabi


def key_offsets(tok_off, block_size: int) -> np.ndarray:
    """key_off[r] = number of keys of requests before r (floor(len / block_size) each); host side."""
    tok_off = np.ascontiguousarray(tok_off, dtype=np.int64)
    out = np.empty(len(tok_off), dtype=np.int64)
    _cabi.call("kvcm_b200_key_offsets", tok_off.ctypes.data_as(ctypes.c_void_p), len(tok_off) - 1, block_size,
               out.ctypes.data_as(ctypes.c_void_p))
    return out


def length_order(tok_off, with_residency: bool = False):
    """Requests sorted by token count, longest first (int32 permutation, host side).  Passing it to
    GenKeyVectorBatch speeds up ragged batches; the keys are the same.  with_residency=True also returns the
    `warps_per_sm` value to pass along (2, 3 or 4 hashing warps per SM when long requests rule the batch, else 0)."""
    tok_off = np.ascontiguousarray(tok_off, dtype=np.int64)
    out = np.empty(len(tok_off) - 1, dtype=np.int32)
    residency = ctypes.c_int32(0)
    _cabi.call("kvcm_b200_length_order", tok_off.ctypes.data_as(ctypes.c_void_p), len(tok_off) - 1,
               out.ctypes.data_as(ctypes.c_void_p), ctypes.byref(residency))
    return (out, residency.value) if with_residency else out


def GenKeyVectorBatch(tokens: torch.Tensor, tok_off: torch.Tensor, block_size: int, key_off: torch.Tensor,
                      n_keys: int, out: torch.Tensor = None, order: torch.Tensor = None,
                      warps_per_sm: int = 0) -> torch.Tensor:
    """Keys of a CSR batch of requests.

    tokens: CUDA tensor of token ids, int32/uint32 (zero-extended) or int64; tok_off / key_off:
    int64 CUDA tensors of n_req + 1 offsets; n_keys = key_off[-1] known on the host; order: optional int32 CUDA
    permutation from length_order().  Returns the int64 key tensor (CSR by key_off).  Asynchronous on the
    current stream."""
    if not tokens.is_cuda:
        raise ValueError("tokens must be a CUDA tensor: this path has no CPU implementation")
    n_req = tok_off.numel() - 1
    tokens, tok_off, key_off = tokens.contiguous(), tok_off.contiguous(), key_off.contiguous()
    if out is None:
        out = torch.empty(max(n_keys, 1), dtype=torch.int64, device=tokens.device)
    if tokens.dtype in (torch.int32, torch.uint32):
        entry = "kvcm_b200_hash_blocks_u32"
    elif tokens.dtype == torch.int64:
        entry = "kvcm_b200_hash_blocks_i64"
    else:
        raise ValueError("token ids must be 32- or 64-bit integers")
    _cabi.bind_device(tokens.device.index)
    with torch.cuda.device(tokens.device):
        _cabi.call(entry, tokens.data_ptr(), tokens.numel(), tok_off.data_ptr(), n_req, block_size, out.data_ptr(),
                   key_off.data_ptr(), order.contiguous().data_ptr() if order is not None else None,
                   warps_per_sm, torch.cuda.current_stream().cuda_stream)
    return out[:n_keys]


def ApplyPrefixHashBatch(hash_ids: torch.Tensor, id_off: torch.Tensor) -> torch.Tensor:
    """One chained key per id; the key CSR equals the id CSR."""
    return GenKeyVectorBatch(hash_ids, id_off, 1, id_off, hash_ids.numel())
