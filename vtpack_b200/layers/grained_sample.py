"""Forward-only counterparts of ``vtpack/layers/grained_sample.py`` with the same
names, argument order and return values (``grained_sample.py:41,81,102`` in the
reference), calling the CUDA kernels through the C ABI."""
import ctypes

import torch

from .. import _lib
from ..runtime import dtype_code, ptr, require_cuda, stream_ptr


def _patches_i32(patches: torch.Tensor) -> torch.Tensor:
    """int32 view of a patch list; the list made by grained_sample_index_to_patch
    carries one so nothing is converted on the way."""
    cached = getattr(patches, "_vtp_i32", None)
    if cached is not None and cached.shape == patches.shape:
        return cached
    return patches.to(torch.int32).contiguous()


def grained_sample_index_to_patch(indices, split_sizes, region_size, num_extra_tokens):
    """indices int [B,Hr,Wr] -> (patches int64 [L,4] on the device, batch_lengths int64 [B]
    on the CPU), as ``grained_sample_index_to_patch`` of the reference
    (``grained_sample.cu:302-345``).  Reading the lengths back synchronises, as it does
    in the reference; the fused block forward never calls this."""
    require_cuda(indices)
    indices = indices.contiguous()
    B, Hr, Wr = indices.shape
    splits = [int(v) for v in split_sizes.tolist()]
    is64 = indices.dtype == torch.int64
    if not is64 and indices.dtype != torch.int32:
        indices = indices.to(torch.int64)
        is64 = True
    dev = indices.device
    l_max = B * (num_extra_tokens + Hr * Wr * max(splits) ** 2)
    counts = torch.empty(B, dtype=torch.int32, device=dev)
    offsets = torch.empty(B + 1, dtype=torch.int32, device=dev)
    p32 = torch.empty(l_max, 4, dtype=torch.int32, device=dev)
    p64 = torch.empty(l_max, 4, dtype=torch.int64, device=dev)
    arr = (ctypes.c_int * len(splits))(*splits)
    _lib.check(_lib.lib().vtp_index_to_patch(
        ptr(indices), 1 if is64 else 0, arr, len(splits), B, Hr, Wr, int(region_size),
        int(num_extra_tokens), ptr(counts), ptr(offsets), ptr(p32), ptr(p64), stream_ptr(dev)))
    batch_lengths = counts.to("cpu", torch.int64)
    L = int(batch_lengths.sum())
    patches = p64[:L]
    patches._vtp_i32 = p32[:L]
    patches._vtp_offsets = offsets
    return patches, batch_lengths


def grained_sample_compress(input, patches, height, width, num_extra_tokens):
    """[B,N,C] -> [L,C] multi-grain mean pooling (``grained_sample.cu:198-239``)."""
    require_cuda(input, patches)
    input = input.contiguous()
    B, N, C = input.shape
    p32 = _patches_i32(patches)
    L = p32.shape[0]
    out = torch.empty(L, C, dtype=input.dtype, device=input.device)
    _lib.check(_lib.lib().vtp_pool(
        ptr(input), dtype_code(input.dtype), B, N, C, int(width), int(num_extra_tokens), ptr(p32), None, L,
        ptr(out), None, None, 0.0, None, None, stream_ptr(input.device)))
    return out


def grained_sample_decompress(input, patches, ref_input, height, width, num_extra_tokens, is_add_ref):
    """[L,C] -> [B,N,C] replicate-unpool, plus ref_input when is_add_ref
    (``grained_sample.cu:241-300``)."""
    require_cuda(input, patches, ref_input)
    input = input.contiguous()
    ref_input = ref_input.contiguous()
    B, N, C = ref_input.shape
    p32 = _patches_i32(patches)
    L = p32.shape[0]
    out = torch.empty(B, N, C, dtype=input.dtype, device=input.device)
    _lib.check(_lib.lib().vtp_unpool_add(
        ptr(input), None, dtype_code(input.dtype), B, N, C, int(width), int(num_extra_tokens), ptr(p32), None,
        L, ptr(ref_input) if is_add_ref else None, ptr(out), stream_ptr(input.device)))
    return out
