"""A second, scalar restatement of the three grained_sample kernels, one work item at a time.

TEST INFRASTRUCTURE ONLY (nothing in the shipped package imports it).  ``dge_oracle.py`` restates
the kernels with vectorised tensor operations; a vectorised restatement can be wrong in a way that
survives look-ups by coordinate (a permuted row order, a transposed sub-patch walk).  The functions
here walk the reference's parallel index space in plain Python loops, one "thread" after the
other, in the order of the statements of the kernels, so that the two restatements check each
other element by element, row order included.  They are meant for small cases.

Each function cites the kernel it follows (paths inside the StevenGrove/vtpack tree).
"""
import numpy as np


def index_to_patch(indices, split_sizes, region_size, num_extra_tokens):
    """``grained_sample_index_to_patch`` host part (``grained_sample.cu:302-345``) and kernel
    (``:146-196``).  indices int [B, Hr, Wr].  Returns (patches int64 [L, 4] with column 2 of the
    extra-token rows left at -7 (the reference never writes it), batch_lengths int64 [B])."""
    indices = np.asarray(indices, dtype=np.int64)
    split_sizes = np.asarray(split_sizes, dtype=np.int64)
    B, Hr, Wr = indices.shape
    sizes = split_sizes[indices]                                  # patch_sizes
    lengths = np.concatenate([np.full((B, 1), num_extra_tokens, np.int64),
                              (sizes * sizes).reshape(B, -1)], axis=1)
    ends = np.cumsum(lengths.reshape(-1))                         # inclusive: where each slot's rows END
    batch_lengths = lengths.sum(1)
    patches = np.full((int(batch_lengths.sum()), 4), -7, np.int64)
    slots = 1 + Hr * Wr
    for item in range(B * slots):                                 # one thread of the kernel each
        b, slot = divmod(item, slots)
        if slot == 0:
            row = ends[item] - num_extra_tokens
            for e in range(num_extra_tokens):
                patches[row, 0], patches[row, 1], patches[row, 3] = b, -e - 1, 1
                row += 1
            continue
        ry, rx = divmod(slot - 1, Wr)
        s = int(sizes[b, ry, rx])
        step = region_size // s
        row = ends[item] - s * s
        for dy in range(s):
            for dx in range(s):
                patches[row] = (b, ry * region_size + dy * step, rx * region_size + dx * step, step)
                row += 1
    return patches, batch_lengths


def compress(x, patches, width, num_extra_tokens):
    """``grained_sample_compress_kernel`` (``grained_sample.cu:31-69``): per (patch, channel) the sum of the
    patch's tokens in (dy, dx) order in the accumulation type, then ONE division by size^2.  x float32
    [B, N, C]."""
    x = np.asarray(x, dtype=np.float32)
    L, C = patches.shape[0], x.shape[2]
    out = np.empty((L, C), np.float32)
    for p in range(L):
        b, y, xs, size = (int(v) for v in patches[p])
        for c in range(C):
            if y < 0:
                out[p, c] = x[b, -y - 1, c]
                continue
            acc = np.float32(0)
            for dy in range(size):
                for dx in range(size):
                    acc = np.float32(acc + x[b, (y + dy) * width + xs + dx + num_extra_tokens, c])
            out[p, c] = np.float32(acc / np.float32(size * size))
    return out


def decompress_add_ref(q, patches, ref, width, num_extra_tokens):
    """``grained_sample_decompress_kernel`` with a reference (``grained_sample.cu:107-144``): every token of a
    patch receives ``q[p] + ref[token]``."""
    q = np.asarray(q, dtype=np.float32)
    ref = np.asarray(ref, dtype=np.float32)
    out = np.full_like(ref, np.nan)
    for p in range(patches.shape[0]):
        b, y, xs, size = (int(v) for v in patches[p])
        for c in range(q.shape[1]):
            if y < 0:
                out[b, -y - 1, c] = np.float32(q[p, c] + ref[b, -y - 1, c])
                continue
            for dy in range(size):
                for dx in range(size):
                    t = (y + dy) * width + xs + dx + num_extra_tokens
                    out[b, t, c] = np.float32(q[p, c] + ref[b, t, c])
    return out
