"""ctypes binding of include/b200_moe.h (the same entry points a Rust `extern "C"` crate binds)."""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libb200moe.so")
_lib = None


class B200Error(RuntimeError):
    """Raised when a library call returns non-zero (mirrors mlx_rs::error::Exception)."""


class QLinear(C.Structure):
    _fields_ = [("weight", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p)]


class MoeConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("hidden", "inter", "n_experts", "top_k", "bits", "group_size",
                                         "router_mode", "norm_topk_prob")]


class MoeParams(C.Structure):
    _fields_ = [("router_weight", C.c_void_p), ("router_logit_bias", C.c_void_p), ("gate_proj", QLinear),
                ("up_proj", QLinear), ("down_proj", QLinear)]


class MoeAux(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("indices", "scores", "perm", "inv_perm", "counts", "offsets", "logits",
                                            "out_f32")]


EXPORTS = {
    # name: (restype, argtypes)
    "b200_last_error": (C.c_char_p, []),
    "b200_set_error_handler": (None, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200_ctx_create": (C.c_int, [C.POINTER(C.c_void_p), C.c_int]),
    "b200_ctx_destroy": (C.c_int, [C.c_void_p]),
    "b200_workspace_bytes": (C.c_int, [C.POINTER(MoeConfig), C.c_int64, C.POINTER(C.c_size_t)]),
    "b200_ctx_reserve": (C.c_int, [C.c_void_p, C.POINTER(MoeConfig), C.c_int64]),
    "b200_ctx_check": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b200_ctx_launch_count": (C.c_int64, [C.c_void_p]),
    "b200_ctx_debug_words": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.c_int]),
    "b200_ctx_set_qmm_path": (C.c_int, [C.c_void_p, C.c_int]),
    "b200_ctx_set_profiling": (C.c_int, [C.c_void_p, C.c_int]),
    "b200_ctx_stage_ms": (C.c_int, [C.c_void_p, C.POINTER(C.c_float), C.c_int]),
    "b200_quantize": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_void_p,
                                C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200_dequantize": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int64,
                                  C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "b200_quantized_matmul": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                        C.c_int, C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    "b200_gather_mm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                 C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    "b200_gather_qmm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                  C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                  C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    "b200_softmax_axis": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p]),
    "b200_argpartition_axis": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p]),
    "b200_take_along_axis": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p,
                                       C.c_void_p]),
    "b200_take_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_int64, C.c_int64, C.c_int64,
                                 C.c_void_p, C.c_void_p]),
    "b200_take_axis": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    "b200_argsort_axis": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p]),
    "b200_topk_axis": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p]),
    "b200_moe_combine": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int64,
                                   C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200_switch_glu_sorted": (C.c_int, [C.c_void_p, C.POINTER(MoeConfig), C.POINTER(MoeParams), C.c_void_p, C.c_void_p,
                                         C.c_int64, C.c_void_p, C.c_void_p]),
    "b200_ep_return_table": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_void_p), C.c_int64,
                                       C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    "b200_switch_glu_sorted_scatter": (C.c_int, [C.c_void_p, C.POINTER(MoeConfig), C.POINTER(MoeParams), C.c_void_p,
                                                 C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    "b200_ep_buffer_alloc": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p), C.c_char_p]),
    "b200_ep_buffer_open": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_void_p)]),
    "b200_ep_buffer_close": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b200_ep_buffer_free": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b200_ep_layout": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_uint32, C.c_void_p, C.c_void_p,
                                 C.c_void_p]),
    "b200_ep_dispatch": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                   C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_void_p), C.c_uint32,
                                   C.c_void_p]),
    "b200_ep_combine": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                  C.c_void_p, C.c_int64, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_uint32, C.c_void_p,
                                  C.c_void_p]),
    "b200_rms_norm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int64, C.c_int64, C.c_void_p,
                                C.c_void_p]),
    "b200_add_rms_norm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int64, C.c_int64,
                                    C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200_add": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    "b200_router_topk": (C.c_int, [C.c_void_p, C.POINTER(MoeConfig), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                   C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200_moe_permute": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_void_p, C.c_void_p]),
    "b200_moe_permute_static": (C.c_int, [C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                          C.c_void_p, C.c_void_p]),
    "b200_switch_glu_forward": (C.c_int, [C.c_void_p, C.POINTER(MoeConfig), C.POINTER(MoeParams), C.c_void_p, C.c_void_p,
                                          C.c_int64, C.c_void_p, C.c_void_p]),
    "b200_ep_comm_create": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_uint32, C.c_uint32,
                                      C.POINTER(C.c_void_p), C.c_char_p]),
    "b200_ep_comm_connect": (C.c_int, [C.c_void_p, C.c_void_p, C.c_char_p]),
    "b200_ep_comm_destroy": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b200_ep_comm_set_chunks": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int]),
    "b200_moe_block_forward_ep": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(MoeConfig), C.POINTER(MoeParams), C.c_void_p,
                                            C.c_int64, C.c_void_p, C.POINTER(MoeAux), C.c_void_p]),
    "b200_moe_block_forward": (C.c_int, [C.c_void_p, C.POINTER(MoeConfig), C.POINTER(MoeParams), C.c_void_p, C.c_int64,
                                         C.c_void_p, C.POINTER(MoeAux), C.c_void_p]),
    "b200_moe_block_forward_prenorm": (C.c_int, [C.c_void_p, C.POINTER(MoeConfig), C.POINTER(MoeParams), C.c_void_p,
                                                 C.c_void_p, C.c_void_p, C.c_float, C.c_int64, C.c_void_p, C.c_void_p,
                                                 C.POINTER(MoeAux), C.c_void_p]),
}


def library_path():
    return _LIB_PATH


def lib():
    """Loads libb200moe.so.  Fails loudly if it has not been built: there is no other code path."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise B200Error(f"{_LIB_PATH} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
                            "(nvcc, sm_100a) first; this package has no fallback implementation")
        l = C.CDLL(_LIB_PATH)
        for name, (res, args) in EXPORTS.items():
            fn = getattr(l, name)  # AttributeError if the header and the library ever drift apart
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


def check(rc):
    if rc != 0:
        raise B200Error(lib().b200_last_error().decode("utf-8", "replace"))


def ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def stream_ptr():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class Context:
    """Owns the library's scratch memory on one device (one per thread, like the reference's streams)."""

    def __init__(self, device=None):
        import torch
        if not torch.cuda.is_available():
            raise B200Error("no CUDA device: this library runs on a B200 only")
        self.device = torch.cuda.current_device() if device is None else int(device)
        h = C.c_void_p()
        check(lib().b200_ctx_create(C.byref(h), self.device))
        self._h = h

    @property
    def handle(self):
        return self._h

    def reserve(self, cfg, max_tokens):
        check(lib().b200_ctx_reserve(self._h, C.byref(cfg), int(max_tokens)))

    @staticmethod
    def workspace_bytes(cfg, max_tokens):
        n = C.c_size_t(0)
        check(lib().b200_workspace_bytes(C.byref(cfg), int(max_tokens), C.byref(n)))
        return int(n.value)

    def check(self):
        check(lib().b200_ctx_check(self._h, stream_ptr()))

    STAGES = ("router_logits", "route_topk", "permute", "prepare_x", "gate_up", "prepare_h", "down", "combine")

    def debug_words(self, n=64):
        buf = (C.c_int32 * n)()
        check(lib().b200_ctx_debug_words(self._h, buf, n))
        return list(buf)

    QMM_AUTO, QMM_SMALL, QMM_TENSOR_CORE = 0, 1, 2

    def set_qmm_path(self, path):
        """Pin the grouped-product kernel (QMM_SMALL / QMM_TENSOR_CORE) or let the library choose (QMM_AUTO)."""
        check(lib().b200_ctx_set_qmm_path(self._h, int(path)))

    def set_profiling(self, on):
        check(lib().b200_ctx_set_profiling(self._h, int(bool(on))))

    def stage_ms(self):
        """Milliseconds of each stage of the last profiled MoeBlock.forward (waits for it)."""
        buf = (C.c_float * len(self.STAGES))()
        check(lib().b200_ctx_stage_ms(self._h, buf, len(self.STAGES)))
        return dict(zip(self.STAGES, [float(v) for v in buf]))

    def launch_count(self):
        return int(lib().b200_ctx_launch_count(self._h))

    def close(self):
        if self._h:
            lib().b200_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_default = {}


def default_context():
    import torch
    d = torch.cuda.current_device() if torch.cuda.is_available() else -1
    if d not in _default:
        _default[d] = Context(d if d >= 0 else None)
    return _default[d]
