"""Python handle on the C++ decode loop (kcb_model_* of the C ABI)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import lib, tiny_model as tm


class _Mat(C.Structure):
    _fields_ = [("blocks", C.c_void_p), ("rows", C.c_int), ("k", C.c_int), ("fmt", C.c_int)]


class _Layer(C.Structure):
    _fields_ = [(n, _Mat) for n in tm.MATS] + [(n, C.c_void_p) for n in ("attn_norm", "ffn_norm", "q_norm", "k_norm")]


class _Desc(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("hidden", "inter", "n_layers", "heads", "kv_heads", "head_dim", "vocab", "max_ctx")] + [
        ("eps", C.c_float), ("rope_base", C.c_float), ("neox", C.c_int), ("qk_norm", C.c_int),
        ("layers", C.POINTER(_Layer)), ("out_norm", C.c_void_p), ("lm_head", _Mat), ("rope_ff", C.c_void_p)]


class Model:
    """Uploads a numpy model (tiny_model.build) to the current GPU and decodes token by token through
    llm::decodeToken on the kc backend."""

    def __init__(self, shape: tm.Shape, model: dict, graphs: int = 1):
        L = lib.raw
        lib.check(L.kcb_init(), "kcb_init")
        self.shape, self._keep = shape, []
        layers = (_Layer * shape.layers)()
        ms = tm.mat_shapes(shape)
        for l, src in enumerate(model["layers"]):
            for name in tm.MATS:
                rows, k, q6 = ms[name]
                setattr(layers[l], name, _Mat(self._ptr(src[name]), rows, k, 6 if q6 else 4))
            layers[l].attn_norm, layers[l].ffn_norm = self._ptr(src["attn_norm"]), self._ptr(src["ffn_norm"])
            if shape.qk_norm:
                layers[l].q_norm, layers[l].k_norm = self._ptr(src["q_norm"]), self._ptr(src["k_norm"])
        d = _Desc()
        for f in ("hidden", "inter", "heads", "kv_heads", "head_dim", "vocab", "max_ctx"):
            setattr(d, f, getattr(shape, f))
        d.n_layers, d.eps, d.rope_base = shape.layers, shape.eps, shape.rope_base
        d.neox, d.qk_norm = int(shape.neox), int(shape.qk_norm)
        d.layers = C.cast(layers, C.POINTER(_Layer))
        d.out_norm = self._ptr(model["out_norm"])
        d.lm_head = _Mat(self._ptr(model["lm_head"]), shape.vocab, shape.hidden, 6)
        self._keep.append(layers)
        self.handle = C.c_void_p()
        st = L.kcb_model_create(C.byref(d), graphs, C.byref(self.handle))
        if st != 0:
            L.kcb_model_last_error.restype = C.c_char_p
            raise RuntimeError(f"kcb_model_create: status {st}: {L.kcb_model_last_error().decode()}")

    @classmethod
    def synthetic(cls, shape: tm.Shape, weights: int, model_seed: int, start_seed: int, graphs: int = 1) -> "Model":
        """llm::buildModels + llm::allocActs: a random-weight model in a synthetic format (weights 0 = Q8, 1 = Q4,
        2 = Q4X8, 3 = Q4X8Q8) with the reference's values for these seeds.  decode() takes token -1."""
        L = lib.raw
        lib.check(L.kcb_init(), "kcb_init")
        self = cls.__new__(cls)
        self.shape, self._keep = shape, []
        d = _Desc()
        for f in ("hidden", "inter", "heads", "kv_heads", "head_dim", "vocab", "max_ctx"):
            setattr(d, f, getattr(shape, f))
        d.n_layers, d.eps, d.rope_base = shape.layers, shape.eps, shape.rope_base
        self.handle = C.c_void_p()
        st = L.kcb_model_create_synthetic(C.byref(d), int(weights), C.c_ulonglong(model_seed), C.c_ulonglong(start_seed), graphs, C.byref(self.handle))
        if st != 0:
            L.kcb_model_last_error.restype = C.c_char_p
            raise RuntimeError(f"kcb_model_create_synthetic: status {st}: {L.kcb_model_last_error().decode()}")
        return self

    def _ptr(self, a):
        a = np.ascontiguousarray(a)
        self._keep.append(a)
        return a.ctypes.data

    def decode(self, token: int, pos: int):
        logits = np.zeros(self.shape.vocab, np.float32)
        arg = C.c_int()
        st = lib.raw.kcb_model_decode(self.handle, token, pos, logits.ctypes.data_as(C.c_void_p), C.byref(arg))
        if st != 0:
            lib.raw.kcb_model_last_error.restype = C.c_char_p
            raise RuntimeError(f"kcb_model_decode: status {st}: {lib.raw.kcb_model_last_error().decode()}")
        return logits, arg.value

    def close(self):
        if self.handle:
            lib.raw.kcb_model_destroy(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


class FastDecoder:
    """The graph-replayed decoder (kcb_decoder_*): one captured CUDA graph replayed per token, position and
    token on the device, fp16 KV cache, greedy pick on the device."""

    def __init__(self, shape: tm.Shape, model: dict, tp=None):
        """tp = (rank, world, exchange_ptrs): the tensor-parallel form; exchange_ptrs[r] is rank r's zero-filled
        exchange area (tp_shared_bytes(shape) bytes) as mapped into this process."""
        L = lib.raw
        self.shape, self._keep = shape, []
        self.rank, self.world = (tp[0], tp[1]) if tp else (0, 1)
        layers = (_Layer * shape.layers)()
        ms = tm.mat_shapes(shape)
        for l, src in enumerate(model["layers"]):
            for name in tm.MATS:
                rows, k, q6 = ms[name]
                setattr(layers[l], name, _Mat(self._ptr(src[name]), rows, k, 6 if q6 else 4))
            layers[l].attn_norm, layers[l].ffn_norm = self._ptr(src["attn_norm"]), self._ptr(src["ffn_norm"])
            if shape.qk_norm:
                layers[l].q_norm, layers[l].k_norm = self._ptr(src["q_norm"]), self._ptr(src["k_norm"])
        d = _Desc()
        for f in ("hidden", "inter", "heads", "kv_heads", "head_dim", "vocab", "max_ctx"):
            setattr(d, f, getattr(shape, f))
        d.n_layers, d.eps, d.rope_base = shape.layers, shape.eps, shape.rope_base
        d.neox, d.qk_norm = int(shape.neox), int(shape.qk_norm)
        d.layers = C.cast(layers, C.POINTER(_Layer))
        d.out_norm = self._ptr(model["out_norm"])
        d.lm_head = _Mat(self._ptr(model["lm_head"]), shape.vocab, shape.hidden, 6)
        self._keep.append(layers)
        self.handle = C.c_void_p()
        if tp:
            ptrs = (C.c_void_p * self.world)(*[int(p) for p in tp[2]])
            st = L.kcb_decoder_create_tp(C.byref(d), int(self.rank), int(self.world), ptrs, C.byref(self.handle))
        else:
            st = L.kcb_decoder_create(C.byref(d), C.byref(self.handle))
        if st != 0:
            L.kcb_decoder_last_error.restype = C.c_char_p
            raise RuntimeError(f"kcb_decoder_create: status {st}: {L.kcb_decoder_last_error().decode()}")
        n, wb = C.c_int(), C.c_longlong()
        L.kcb_decoder_info(self.handle, C.byref(n), C.byref(wb))
        self.launches_per_token, self.weight_bytes = n.value, wb.value
        self._keep.clear()  # weights now live on the device

    def _ptr(self, a):
        a = np.ascontiguousarray(a)
        self._keep.append(a)
        return a.ctypes.data

    @staticmethod
    def tp_shared_bytes(shape: tm.Shape) -> int:
        d = _Desc()
        d.hidden = shape.hidden
        lib.raw.kcb_decoder_tp_shared_bytes.restype = C.c_size_t
        return int(lib.raw.kcb_decoder_tp_shared_bytes(C.byref(d)))

    @staticmethod
    def tp_timeouts() -> int:
        lib.raw.kcb_decoder_tp_timeouts.restype = C.c_uint
        return int(lib.raw.kcb_decoder_tp_timeouts())

    def local_rows(self):
        """Rows of the logits this rank fills (all of them on one GPU)."""
        per = self.shape.vocab // self.world
        return self.rank * per, (self.rank + 1) * per

    def set_prompt(self, tokens, start_pos=0):
        t = np.ascontiguousarray(tokens, np.int32)
        lib.check(lib.raw.kcb_decoder_set_prompt(self.handle, t.ctypes.data_as(C.c_void_p), int(t.size), int(start_pos)), "kcb_decoder_set_prompt")

    def prefill(self, tokens, start_pos=0):
        """Batched prompt pass (one GPU, or tensor parallel with whole-super-block shares): returns once the KV cache holds the prompt and the first pick is made."""
        t = np.ascontiguousarray(tokens, np.int32)
        st = lib.raw.kcb_decoder_prefill(self.handle, t.ctypes.data_as(C.c_void_p), int(t.size), int(start_pos))
        if st != 0:
            lib.raw.kcb_decoder_last_error.restype = C.c_char_p
            raise lib.KcbError("kcb_decoder_prefill", st, lib.raw.kcb_decoder_last_error().decode())

    # ---- a batch of independent sequences in lockstep ----
    def batch_begin(self, n_sequences: int):
        self._batch_call(lib.raw.kcb_decoder_batch_begin(self.handle, int(n_sequences)), "kcb_decoder_batch_begin")

    def batch_prefill(self, seq: int, tokens):
        t = np.ascontiguousarray(tokens, np.int32)
        self._batch_call(lib.raw.kcb_decoder_batch_prefill(self.handle, int(seq), t.ctypes.data_as(C.c_void_p), int(t.size)), "kcb_decoder_batch_prefill")

    def batch_run(self, steps: int):
        self._batch_call(lib.raw.kcb_decoder_batch_run(self.handle, int(steps)), "kcb_decoder_batch_run")

    def batch_read(self, seq: int, n_history=0):
        logits = np.zeros(self.shape.vocab, np.float32)
        hist = np.zeros(max(n_history, 1), np.int32)
        pos = C.c_int()
        self._batch_call(lib.raw.kcb_decoder_batch_read(self.handle, int(seq), logits.ctypes.data_as(C.c_void_p), hist.ctypes.data_as(C.c_void_p),
                                                        int(n_history), C.byref(pos)), "kcb_decoder_batch_read")
        return logits, hist[:n_history], pos.value

    def _batch_call(self, st, what):
        if st != 0:
            lib.raw.kcb_decoder_last_error.restype = C.c_char_p
            raise lib.KcbError(what, st, lib.raw.kcb_decoder_last_error().decode())

    def run(self, steps: int):
        lib.check(lib.raw.kcb_decoder_run(self.handle, int(steps)), "kcb_decoder_run")

    def sync(self):
        lib.check(lib.raw.kcb_decoder_sync(self.handle), "kcb_decoder_sync")

    def read(self, n_history=0, want_logits=True):
        logits = np.zeros(self.shape.vocab, np.float32) if want_logits else None
        hist = np.zeros(max(n_history, 1), np.int32)
        pos = C.c_int()
        lib.check(lib.raw.kcb_decoder_read(self.handle, logits.ctypes.data_as(C.c_void_p) if want_logits else None,
                                           hist.ctypes.data_as(C.c_void_p), int(n_history), C.byref(pos)), "kcb_decoder_read")
        return logits, hist[:n_history], pos.value

    def enable_trace(self) -> int:
        """Test instrumentation: every later step keeps the int8 words of each activation vector it quantizes and the
        residual stream after each addition (layout: include/kernelcore_b200.h, kcb_decoder_enable_trace).  Returns
        the int32 words per step."""
        n = C.c_size_t()
        lib.check(lib.raw.kcb_decoder_enable_trace(self.handle, C.byref(n)), "kcb_decoder_enable_trace")
        self._trace_words = n.value
        return n.value

    def read_trace(self) -> np.ndarray:
        out = np.zeros(self._trace_words, np.int32)
        lib.check(lib.raw.kcb_decoder_read_trace(self.handle, out.ctypes.data_as(C.c_void_p), C.c_size_t(out.size)), "kcb_decoder_read_trace")
        return out

    @property
    def cuda_stream(self) -> int:
        lib.raw.kcb_decoder_stream.restype = C.c_void_p
        return lib.raw.kcb_decoder_stream(self.handle) or 0

    def close(self):
        if self.handle:
            lib.raw.kcb_decoder_destroy(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()
