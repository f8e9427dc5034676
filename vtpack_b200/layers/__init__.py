"""Drop-in for ``vtpack.layers``, backed by libvtpack_b200.so."""
from .bilinear_attention import bilinear_attention, sparse_bilinear_attention_pointwise_forward
from .dge import DynamicGrainedEncoder, DynamicRouter
from .grained_sample import (
    grained_sample_compress,
    grained_sample_decompress,
    grained_sample_index_to_patch,
)
from .sparse_ops import batched_sparse_attention, batched_sparse_gemm

__all__ = [
    "DynamicGrainedEncoder", "DynamicRouter", "grained_sample_compress", "grained_sample_decompress",
    "grained_sample_index_to_patch", "batched_sparse_attention", "batched_sparse_gemm", "bilinear_attention",
    "sparse_bilinear_attention_pointwise_forward",
]
