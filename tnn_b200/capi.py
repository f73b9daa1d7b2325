"""ctypes binding of the C ABI declared in include/tnn_b200.h.

The library is the product: if `tnn_b200/lib/libtnn_b200.so` is missing this module raises — there is no fallback.
Tensors are torch CUDA tensors used purely as device buffers; every call goes through the `extern "C"` entry points
with raw pointers and the current torch stream.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("TNN_B200_LIB", os.path.join(_HERE, "lib", "libtnn_b200.so"))

F16, BF16, F32 = 0, 1, 2
EPI_BIAS, EPI_BIAS_GELU, EPI_BIAS_RESIDUAL, EPI_BIAS_TANH = 0, 1, 2, 3

OK = 0
ERR_PARAM, ERR_UNSUPPORTED, ERR_LAUNCH, ERR_DRIVER, ERR_DEVICE_TIMEOUT, ERR_NOT_SM100 = -1, -2, -3, -4, -5, -6
ERR_STATIC_LIMIT = -7
ERR_INDEX = -8
STATIC_MAX_BATCH = 4096

_c = ctypes
_i64, _i32, _f32, _vp = _c.c_int64, _c.c_int32, _c.c_float, _c.c_void_p


class LinearDesc(_c.Structure):
    _fields_ = [("x", _vp), ("w_nk", _vp), ("bias", _vp), ("residual", _vp), ("y", _vp),
                ("M", _i64), ("N", _i64), ("K", _i64),
                ("ldx", _i64), ("ldw", _i64), ("ldr", _i64), ("ldy", _i64),
                ("dtype", _i32), ("out_dtype", _i32), ("epilogue", _i32), ("block_n", _i32),
                ("out_stats", _vp), ("ln_in_stats", _vp), ("ln_c1", _vp), ("ln_c2", _vp),
                ("res_ln_stats", _vp), ("res_ln_gamma", _vp), ("res_ln_beta", _vp),
                ("ln_eps", _f32), ("reserved_", _i32)]


class AttentionDesc(_c.Structure):
    _fields_ = [("q", _vp), ("k", _vp), ("v", _vp), ("mask_add", _vp), ("kv_len", _vp), ("out", _vp),
                ("B", _i64), ("S", _i64),
                ("ldq", _i64), ("ldk", _i64), ("ldv", _i64), ("ldo", _i64),
                ("heads", _i32), ("head_dim", _i32), ("dtype", _i32),
                ("scale", _f32), ("mask_exclude_below", _f32)]


class LayerNormDesc(_c.Structure):
    _fields_ = [("x", _vp), ("residual", _vp), ("gamma", _vp), ("beta", _vp), ("y", _vp),
                ("rows", _i64), ("H", _i64),
                ("ldx", _i64), ("ldr", _i64), ("ldy", _i64),
                ("in_dtype", _i32), ("out_dtype", _i32), ("eps", _f32)]


class EmbeddingDesc(_c.Structure):
    _fields_ = [("input_ids", _vp), ("segment_ids", _vp), ("word_emb", _vp), ("type_emb", _vp), ("pos_emb", _vp),
                ("gamma", _vp), ("beta", _vp), ("out", _vp),
                ("B", _i64), ("S", _i64), ("H", _i64), ("vocab", _i64), ("type_vocab", _i64),
                ("ld_table", _i64), ("ld_out", _i64),
                ("table_dtype", _i32), ("out_dtype", _i32), ("eps", _f32)]


class QAHeadDesc(_c.Structure):
    _fields_ = [("x", _vp), ("weight", _vp), ("bias", _vp), ("out", _vp),
                ("M", _i64), ("H", _i64), ("ldx", _i64), ("ld_out", _i64),
                ("N", _i32), ("x_dtype", _i32), ("out_n", _vp * 4)]


class EncoderLayerWeights(_c.Structure):
    _fields_ = [("w_qkv", _vp), ("b_qkv", _vp), ("w_o", _vp), ("b_o", _vp),
                ("ln1_gamma", _vp), ("ln1_beta", _vp),
                ("w_ffn1", _vp), ("b_ffn1", _vp), ("w_ffn2", _vp), ("b_ffn2", _vp),
                ("ln2_gamma", _vp), ("ln2_beta", _vp),
                ("qkv_c1", _vp), ("qkv_c2", _vp), ("ffn1_c1", _vp), ("ffn1_c2", _vp)]


class EncoderDesc(_c.Structure):
    _fields_ = [("hidden", _vp), ("mask_add", _vp), ("kv_len", _vp), ("layers", _c.POINTER(EncoderLayerWeights)),
                ("workspace", _vp),
                ("B", _i64), ("S", _i64), ("H", _i64), ("F", _i64),
                ("heads", _i32), ("num_layers", _i32), ("dtype", _i32),
                ("ln_eps", _f32), ("mask_exclude_below", _f32), ("fold_layernorm", _i32)]


# name -> (restype, argtypes); every symbol include/tnn_b200.h declares
SYMBOLS = {
    "b200_pack_weight": (_c.c_int, [_vp, _i64, _i64, _i64, _vp, _i64, _c.c_int, _vp]),
    "b200_fold_layernorm_weight": (_c.c_int, [_vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _i64, _c.c_int, _vp, _vp, _vp]),
    "b200_convert": (_c.c_int, [_vp, _c.c_int, _vp, _c.c_int, _i64, _vp]),
    "b200_linear_fwd": (_c.c_int, [_c.POINTER(LinearDesc), _vp]),
    "b200_attention_fwd": (_c.c_int, [_c.POINTER(AttentionDesc), _vp]),
    "b200_attention_masked_fwd_static": (_c.c_int, [_c.POINTER(AttentionDesc), _vp]),
    "b200_mask_to_kv_len": (_c.c_int, [_vp, _i64, _i64, _f32, _vp, _vp]),
    "b200_add_layernorm_fwd": (_c.c_int, [_c.POINTER(LayerNormDesc), _vp]),
    "b200_embedding_layernorm_fwd": (_c.c_int, [_c.POINTER(EmbeddingDesc), _vp]),
    "b200_mask_from_input_mask": (_c.c_int, [_vp, _i64, _i64, _f32, _f32, _vp, _vp, _vp]),
    "b200_qa_head_fwd": (_c.c_int, [_c.POINTER(QAHeadDesc), _vp]),
    "b200_encoder_workspace_bytes": (_c.c_size_t, [_i64, _i64, _i64, _c.c_int]),
    "b200_encoder_fwd": (_c.c_int, [_c.POINTER(EncoderDesc), _vp]),
    "b200_status_string": (_c.c_char_p, [_c.c_int]),
    "b200_device_status": (_c.c_int, []),
    "b200_device_status_async": (_c.c_int, [_vp, _vp]),
    "b200_decode_status_word": (_c.c_int, [_c.c_uint]),
    "b200_launch_count": (_c.c_uint64, []),
    "b200_version": (_c.c_char_p, []),
    "b200_selftest_bounded_wait": (_c.c_int, [_vp]),
    "b200_selftest_tensor_map_cache": (_c.c_int, [_c.c_int, _c.c_int, _c.c_int]),
}

_lib = None


class B200Error(RuntimeError):
    def __init__(self, code, where):
        self.code = code
        try:
            msg = lib().b200_status_string(code).decode()
        except Exception:  # pragma: no cover
            msg = "?"
        super().__init__("%s failed: %d (%s)" % (where, code, msg))


def lib():
    """Load the CUDA kernel library; raise if it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError("tnn_b200 CUDA library missing at %s: run `python -m tnn_b200.build`" % LIB_PATH)
        l = _c.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(l, name)  # AttributeError if the library does not export a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


def check(code, where):
    if code != OK:
        raise B200Error(code, where)


def dtype_code(dt):
    if dt == torch.float16:
        return F16
    if dt == torch.bfloat16:
        return BF16
    if dt == torch.float32:
        return F32
    raise ValueError("unsupported dtype %s" % dt)


def torch_dtype(code):
    return {F16: torch.float16, BF16: torch.bfloat16, F32: torch.float32}[code]


def ptr(t):
    return None if t is None else t.data_ptr()


def stream_ptr():
    return torch.cuda.current_stream().cuda_stream


def device_status():
    return lib().b200_device_status()


def launch_count():
    return int(lib().b200_launch_count())
