"""ctypes binding of libvtpack_b200.so (the C ABI declared in include/vtpack_b200.h).

There is no CPU or PyTorch fallback: if the library has not been built,
importing the ops raises with the build command.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libvtpack_b200.so")

VTP_F32, VTP_BF16 = 0, 1
FLAG_GELU, FLAG_OUT_F32, FLAG_CUDA_CORES = 1, 2, 4
# return codes (include/vtpack_b200.h) and the index-guard bit of the device status word
ERR_NULL, ERR_SHAPE, ERR_DTYPE, ERR_ALIGN, ERR_UNSUPPORTED, ERR_DRIVER = -1, -2, -3, -4, -5, -6
STATUS_BAD_INDEX = 64

c_void_p, c_int, c_ll, c_float, c_uint = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_uint


class BlockWeights(C.Structure):
    _fields_ = [(n, c_void_p) for n in (
        "norm1_w", "norm1_b", "q_w", "q_b", "kv_w", "kv_b", "proj_w", "proj_b",
        "norm2_w", "norm2_b", "fc1_w", "fc1_b", "fc2_w", "fc2_b", "gate_w", "gate_b",
        "q_wf", "q_s", "q_c", "kv_wf", "kv_s", "kv_c", "fc1_wf", "fc1_s", "fc1_c",
        "sr_w", "sr_b", "sr_norm_w", "sr_norm_b")]


class DgeShape(C.Structure):
    _fields_ = [("dtype", c_int), ("B", c_int), ("H", c_int), ("W", c_int), ("num_extra", c_int),
                ("C", c_int), ("heads", c_int), ("hidden", c_int), ("region", c_int),
                ("n_splits", c_int), ("splits", c_int * 8), ("eps", c_float), ("flags", c_uint),
                ("sr_ratio", c_int), ("sr_eps", c_float), ("attn_scale", c_float)]


class ModelWeights(C.Structure):
    _fields_ = [("patch_w", c_void_p), ("patch_b", c_void_p), ("cls_token", c_void_p),
                ("pos_embed", c_void_p), ("norm_w", c_void_p), ("norm_b", c_void_p),
                ("head_w", c_void_p), ("head_b", c_void_p), ("depth", c_int), ("patch", c_int),
                ("img_size", c_int), ("num_classes", c_int), ("image_dtype", c_int)]


class ForwardOptions(C.Structure):
    _fields_ = [("gate_image_bias", c_void_p), ("tokens_trace", c_void_p), ("grain_trace", c_void_p)]


# name -> (restype, argtypes); every symbol include/vtpack_b200.h declares
PROTOTYPES = {
    "vtp_version": (c_int, []),
    "vtp_last_error_string": (C.c_char_p, []),
    "vtp_device_status": (c_int, [C.POINTER(c_int), c_int]),
    "vtp_router_gate": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "vtp_gate_argmax": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "vtp_index_to_patch": (c_int, [c_void_p, c_int, C.POINTER(c_int), c_int, c_int, c_int, c_int, c_int,
                                   c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "vtp_gate_compact_static": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                        c_void_p, C.POINTER(c_int), c_int, c_void_p, c_void_p, c_void_p]),
    "vtp_pool": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                         c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p]),
    "vtp_unpool_add": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                               c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "vtp_pool_grad": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                              c_void_p, c_void_p]),
    "vtp_unpool_grad": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                                c_void_p, c_void_p]),
    "vtp_region_layout_supported": (c_int, [c_int, c_int]),
    "vtp_unpool_grad_regions": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                        C.POINTER(c_int), c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "vtp_batched_sparse_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_ll, c_int, c_ll,
                                        c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_ll, c_int,
                                        c_void_p]),
    "vtp_bilinear_attention_forward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                               c_int, c_int, c_int, c_int, c_void_p]),
    "vtp_sparse_bilinear_attention_forward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                                      c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "vtp_bilinear_attention_backward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                c_void_p]),
    "vtp_layernorm": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_ll, c_void_p, c_void_p, c_float,
                              c_void_p, c_void_p]),
    "vtp_token_im2col": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "vtp_add_rows": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_ll,
                             c_int, c_void_p]),
    "vtp_linear": (c_int, [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_void_p, c_ll, c_int,
                           c_int, c_void_p, c_int, c_int, c_uint, c_void_p]),
    "vtp_fold_layernorm": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_void_p]),
    "vtp_sparse_attention": (c_int, [c_void_p, c_ll, c_ll, c_void_p, c_void_p, c_ll, c_ll, c_ll, c_void_p,
                                     c_ll, c_ll, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                     c_int, c_float, c_uint, c_void_p]),
    "vtp_patch_im2col": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                 c_int, c_void_p, c_void_p]),
    "vtp_layernorm_add_rows": (c_int, [c_void_p, c_int, c_int, c_int, c_ll, c_void_p, c_void_p, c_float, c_void_p, c_int,
                                       c_int, c_void_p, c_int, c_int, c_int, c_void_p]),
    "vtp_patch_im2col_padded": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p]),
    "vtp_block_workspace_bytes": (c_ll, [C.POINTER(DgeShape)]),
    "vtp_dge_block_forward": (c_int, [C.POINTER(DgeShape), C.POINTER(BlockWeights), c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_ll, c_void_p]),
    "vtp_dge_blocks_forward": (c_int, [C.POINTER(DgeShape), C.POINTER(BlockWeights), c_int, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_ll, c_void_p]),
    "vtp_dge_block_forward_timed": (c_int, [C.POINTER(DgeShape), C.POINTER(BlockWeights), c_void_p, c_void_p,
                                            c_void_p, c_void_p, c_void_p, c_ll, C.POINTER(c_void_p), c_int,
                                            c_void_p]),
    "vtp_dense_block_forward": (c_int, [C.POINTER(DgeShape), C.POINTER(BlockWeights), c_void_p, c_void_p,
                                        c_void_p, c_ll, c_void_p]),
    "vtp_model_workspace_bytes": (c_ll, [C.POINTER(DgeShape), C.POINTER(ModelWeights)]),
    "vtp_deit_dge_forward": (c_int, [C.POINTER(DgeShape), C.POINTER(ModelWeights), C.POINTER(BlockWeights),
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_void_p]),
    "vtp_deit_dge_forward_ex": (c_int, [C.POINTER(DgeShape), C.POINTER(ModelWeights), C.POINTER(BlockWeights),
                                        c_void_p, c_void_p, c_void_p, C.POINTER(ForwardOptions), c_void_p, c_ll,
                                        c_void_p]),
}

_lib = None


def lib():
    """The loaded library.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m vtpack_b200.build` "
                "(needs nvcc; there is no CPU or PyTorch fallback)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


class VtpError(RuntimeError):
    def __init__(self, code, text):
        super().__init__(f"vtpack_b200 error {code}: {text}")
        self.code = code


def check(rc):
    if rc != 0:
        raise VtpError(rc, lib().vtp_last_error_string().decode("utf-8", "replace"))


def device_status(reset=True):
    v = c_int(0)
    check(lib().vtp_device_status(C.byref(v), 1 if reset else 0))
    return v.value
