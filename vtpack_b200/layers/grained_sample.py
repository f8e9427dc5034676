"""Counterparts of ``vtpack/layers/grained_sample.py`` with the same names, argument order and
return values (``grained_sample.py:41,81,102`` in the reference), calling the CUDA kernels through
the C ABI.  ``grained_sample_compress`` and ``grained_sample_decompress`` are differentiable: their
backward passes are the gradient kernels ``vtp_pool_grad`` / ``vtp_unpool_grad``
(``grained_sample.py:26-38`` and ``:61-78``)."""
import ctypes

import torch
from torch.autograd import Function
from torch.autograd.function import once_differentiable

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
    # what the region-parallel gradient kernel needs instead of the list: the grain index of every region and
    # the packed row of its first patch (the image's first row + its extra tokens + the patches of the regions
    # in front of it)
    per_side = torch.tensor(splits, dtype=torch.int32, device=dev)[indices.reshape(B, -1).clamp(0, len(splits) - 1)]
    per_region = per_side * per_side
    first = offsets[:B, None] + int(num_extra_tokens) + torch.cumsum(per_region, 1, dtype=torch.int32) - per_region
    patches._vtp_regions = (indices.reshape(B, -1).to(torch.int32).contiguous(), first.to(torch.int32).contiguous(),
                            splits, int(region_size), Hr, Wr, int(num_extra_tokens))
    return patches, batch_lengths


def _mover_args(t, p32, width, num_extra_tokens):
    B, N, C = t
    return (B, N, C, int(width), int(num_extra_tokens), ptr(p32), None, p32.shape[0])


class _GrainedSampleCompress(Function):
    """[B,N,C] -> [L,C] multi-grain mean pooling (``grained_sample.cu:198-239``); the gradient
    hands every token 1/size^2 of its patch's row (``grained_sample.py:26-38``)."""

    @staticmethod
    def forward(ctx, input, patches, height, width, num_extra_tokens):
        require_cuda(input, patches)
        input = input.contiguous()
        p32 = _patches_i32(patches)
        ctx.save_for_backward(p32)
        ctx.geom = (tuple(input.shape), int(width), int(num_extra_tokens))
        out = torch.empty(p32.shape[0], input.shape[2], dtype=input.dtype, device=input.device)
        _lib.check(_lib.lib().vtp_pool(
            ptr(input), dtype_code(input.dtype), *_mover_args(input.shape, p32, width, num_extra_tokens),
            ptr(out), None, None, 0.0, None, None, stream_ptr(input.device)))
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        p32, = ctx.saved_tensors
        shape, width, num_extra_tokens = ctx.geom
        grad_output = grad_output.contiguous()
        grad_input = torch.empty(shape, dtype=grad_output.dtype, device=grad_output.device)
        _lib.check(_lib.lib().vtp_pool_grad(
            ptr(grad_output), dtype_code(grad_output.dtype), *_mover_args(shape, p32, width, num_extra_tokens),
            ptr(grad_input), stream_ptr(grad_output.device)))
        return grad_input, None, None, None, None


class _GrainedSampleDecompress(Function):
    """[L,C] -> [B,N,C] replicate-unpool, plus ref_input when is_add_ref
    (``grained_sample.cu:241-300``); the gradient of the packed rows is the sum over each patch's
    tokens, that of ref_input the incoming gradient or zero (``grained_sample.py:61-78``)."""

    @staticmethod
    def forward(ctx, input, patches, ref_input, height, width, num_extra_tokens, is_add_ref):
        require_cuda(input, patches, ref_input)
        input = input.contiguous()
        ref_input = ref_input.contiguous()
        p32 = _patches_i32(patches)
        ctx.save_for_backward(p32)
        ctx.geom = (tuple(ref_input.shape), int(width), int(num_extra_tokens), bool(is_add_ref))
        ctx.regions = (getattr(patches, "_vtp_regions", None), getattr(patches, "_vtp_offsets", None))
        out = torch.empty(ref_input.shape, dtype=input.dtype, device=input.device)
        B, N, C = ref_input.shape
        _lib.check(_lib.lib().vtp_unpool_add(
            ptr(input), None, dtype_code(input.dtype), *_mover_args(ref_input.shape, p32, width, num_extra_tokens),
            ptr(ref_input) if is_add_ref else None, ptr(out), stream_ptr(input.device)))
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        p32, = ctx.saved_tensors
        shape, width, num_extra_tokens, is_add_ref = ctx.geom
        grad_output = grad_output.contiguous()
        grad_input = torch.empty(p32.shape[0], shape[2], dtype=grad_output.dtype, device=grad_output.device)
        lib = _lib.lib()
        regions, offsets = ctx.regions
        B, N, C = shape
        if (regions is not None and offsets is not None and regions[3] == 4 and regions[6] == num_extra_tokens
                and regions[0].shape[0] == B and N == num_extra_tokens + regions[4] * regions[5] * 16
                and width == regions[5] * 4 and lib.vtp_region_layout_supported(dtype_code(grad_output.dtype), C)):
            # the list came from grain indices: one thread block per region instead of a walk over the list
            idx32, first, splits, region_size, Hr, Wr, _ = regions
            arr = (ctypes.c_int * len(splits))(*splits)
            _lib.check(lib.vtp_unpool_grad_regions(
                ptr(grad_output), dtype_code(grad_output.dtype), B, Hr, Wr, region_size, C, num_extra_tokens,
                ptr(idx32), arr, len(splits), ptr(first), ptr(offsets), p32.shape[0], ptr(grad_input),
                stream_ptr(grad_output.device)))
        else:
            _lib.check(lib.vtp_unpool_grad(
                ptr(grad_output), dtype_code(grad_output.dtype), *_mover_args(shape, p32, width, num_extra_tokens),
                ptr(grad_input), stream_ptr(grad_output.device)))
        grad_ref = grad_output if is_add_ref else torch.zeros_like(grad_output)
        return grad_input, None, grad_ref, None, None, None, None


grained_sample_compress = _GrainedSampleCompress.apply
grained_sample_decompress = _GrainedSampleDecompress.apply


def grained_sample_compress_dense(x, split_sizes, region_size, H, W, num_extra_tokens):
    """Every grain of every region, for dense training: [B,N,C] -> ([B*(extra + sum_k (H/step_k)(W/step_k)), C],
    batch_lengths), per image [extra | grain split_sizes[0] | split_sizes[1] | ...]
    (``grained_sample.py:126-147``).  Plain tensor algebra, differentiable through autograd."""
    B, N, C = x.shape
    grid = x[:, num_extra_tokens:, :].reshape(B, H, W, C)
    parts = [x[:, :num_extra_tokens, :]] if num_extra_tokens > 0 else []
    for win in split_sizes.tolist():
        step = region_size // int(win)
        parts.append(grid.reshape(B, H // step, step, W // step, step, C).mean(dim=(2, 4)).reshape(B, -1, C))
    comp = torch.cat(parts, dim=1)
    batches = torch.full([B], comp.shape[1], dtype=torch.long)
    return comp.reshape(-1, C), batches


def grained_sample_decompress_dense(x, gate, reference, split_sizes, region_size, H, W, num_extra_tokens,
                                    is_add_ref):
    """Inverse of the dense layout: every grain replicated back to the token grid, weighted by its
    (one-hot, straight-through) gate value and summed (``grained_sample.py:150-177``)."""
    B, N, C = reference.shape
    Hr, Wr = gate.shape[1:3]
    x = x.reshape(B, -1, C)
    out = None
    start = num_extra_tokens
    for i, win in enumerate(split_sizes.tolist()):
        step = region_size // int(win)
        Hi, Wi = H // step, W // step
        rows = x[:, start:start + Hi * Wi, :].reshape(B, Hi, 1, Wi, 1, C).expand(B, Hi, step, Wi, step, C)
        rows = rows.reshape(B, Hr, H // Hr, Wr, W // Wr, C)
        term = (rows * gate[..., i].reshape(B, Hr, 1, Wr, 1, 1)).reshape(B, H * W, C)
        out = term if out is None else out + term
        start += Hi * Wi
    if num_extra_tokens > 0:
        out = torch.cat([x[:, :num_extra_tokens, :], out], dim=1)
    return out + reference if is_add_ref else out
