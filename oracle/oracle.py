"""ctypes view of the CPU oracle (oracle/liboracle.so).

TEST INFRASTRUCTURE ONLY: the oracle restates the reference's Rust sampler chain in C and is
the checker for the CUDA path.  Only the test-suite, the smoke check and the CPU-baseline
leg of the benchmark import this module; the shipped package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

ROW_OK, ROW_NONFINITE, ROW_DEAD, ROW_EMPTY = 0, 1, 2, 3


def build(force: bool = False) -> str:
    """Compile oracle/*.c with the Makefile beside it."""
    srcs = [os.path.join(_HERE, f) for f in ("pagoda_oracle.c", "pagoda_oracle_grammar.c", "pagoda_oracle.h")]
    stale = force or not os.path.exists(_LIB_PATH) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in srcs)
    if stale:
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


class RowParams(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("top_k", C.c_uint32),
                ("freq", C.c_float), ("pres", C.c_float), ("rep", C.c_float),
                ("history", C.POINTER(C.c_uint32)), ("n_history", C.c_uint32),
                ("mask_words", C.POINTER(C.c_uint32)), ("grammar_dead", C.c_int),
                ("grammar_complete", C.c_int), ("eos_id", C.c_int32), ("uniform", C.c_float)]


class RowOut(C.Structure):
    _fields_ = [("token", C.c_uint32), ("status", C.c_int32), ("drew", C.c_int32),
                ("argmax", C.c_uint32), ("row_max", C.c_float), ("sumexp", C.c_float),
                ("total", C.c_float), ("n_kept", C.c_uint32), ("margin", C.c_float),
                ("margin_k", C.c_float), ("margin_p", C.c_float), ("margin_cdf", C.c_float)]


class Batch(C.Structure):
    _fields_ = [("logits", C.POINTER(C.c_float)), ("rows", C.c_size_t), ("vocab", C.c_size_t),
                ("row_stride", C.c_size_t),
                ("temperature", C.POINTER(C.c_float)), ("top_p", C.POINTER(C.c_float)),
                ("top_k", C.POINTER(C.c_uint32)),
                ("freq", C.POINTER(C.c_float)), ("pres", C.POINTER(C.c_float)), ("rep", C.POINTER(C.c_float)),
                ("hist_offsets", C.POINTER(C.c_uint32)), ("hist_ids", C.POINTER(C.c_uint32)),
                ("mask_rows", C.POINTER(C.POINTER(C.c_uint32))), ("row_flags", C.POINTER(C.c_uint8)),
                ("eos_id", C.c_int32), ("uniform", C.POINTER(C.c_float))]


class TpOut(C.Structure):
    _fields_ = [("token", C.c_uint32), ("status", C.c_int32), ("drew", C.c_int32), ("argmax", C.c_uint32),
                ("gmax", C.c_float), ("gsum", C.c_float), ("total", C.c_float), ("n_kept", C.c_uint32),
                ("margin", C.c_float)]


ROW_OUT_DTYPE = np.dtype([("token", "<u4"), ("status", "<i4"), ("drew", "<i4"), ("argmax", "<u4"),
                          ("row_max", "<f4"), ("sumexp", "<f4"), ("total", "<f4"), ("n_kept", "<u4"),
                          ("margin", "<f4"), ("margin_k", "<f4"), ("margin_p", "<f4"), ("margin_cdf", "<f4")])

_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        fp, u32p, u8p = C.POINTER(C.c_float), C.POINTER(C.c_uint32), C.POINTER(C.c_uint8)
        L.pgo_rng_next_u64.restype = C.c_uint64
        L.pgo_rng_next_f64.restype = C.c_double
        L.pgo_rng_next_f32.restype = C.c_float
        L.pgo_argmax.restype = C.c_uint32
        L.pgo_argmax.argtypes = [fp, C.c_size_t]
        L.pgo_log_softmax.argtypes = [fp, C.c_size_t, fp]
        L.pgo_temperature_softmax.argtypes = [fp, C.c_size_t, C.c_float]
        L.pgo_apply_top_k.argtypes = [fp, C.c_size_t, C.c_uint64]
        L.pgo_apply_top_p.argtypes = [fp, C.c_size_t, C.c_float]
        L.pgo_sample_categorical.restype = C.c_uint32
        L.pgo_sample_categorical.argtypes = [fp, C.c_size_t, C.c_float, C.POINTER(C.c_int)]
        L.pgo_sample.restype = C.c_uint32
        L.pgo_sample.argtypes = [fp, C.c_size_t, C.c_float, C.c_uint64, C.c_float, C.c_float, C.POINTER(C.c_int)]
        L.pgo_logits_sane.argtypes = [fp, C.c_size_t, C.c_size_t]
        L.pgo_apply_penalties.argtypes = [fp, C.c_size_t, u32p, C.c_size_t, C.c_float, C.c_float]
        L.pgo_apply_repetition.argtypes = [fp, C.c_size_t, u32p, C.c_size_t, C.c_float]
        L.pgo_mask_logits_bytes.argtypes = [u8p, C.c_size_t, fp, C.c_size_t]
        L.pgo_mask_logits_bits.argtypes = [u32p, fp, C.c_size_t]
        L.pgo_sample_row.argtypes = [fp, C.c_size_t, C.POINTER(RowParams), C.POINTER(RowOut), fp, fp]
        L.pgo_sample_batch.argtypes = [C.POINTER(Batch), C.c_void_p, C.c_int]
        L.pgo_bf16_to_f32.argtypes = [C.POINTER(C.c_uint16), fp, C.c_size_t]
        L.pgo_tp_sample_row.argtypes = [fp, C.c_size_t, C.c_uint32, C.c_uint32, C.POINTER(RowParams),
                                        C.POINTER(TpOut)]
        L.pgo_draft_accept.restype = C.c_uint32
        L.pgo_draft_accept.argtypes = [u32p, u32p, C.c_uint32, u32p]
        L.pgo_regex_new.restype = C.c_void_p
        L.pgo_regex_new.argtypes = [C.c_char_p, C.c_char_p, C.c_size_t]
        L.pgo_regex_free.argtypes = [C.c_void_p]
        L.pgo_regex_is_complete.argtypes = [C.c_void_p, C.c_char_p, C.c_size_t]
        L.pgo_regex_allowed_bytes.argtypes = [C.c_void_p, C.c_char_p, C.c_size_t, u8p]
        L.pgo_json_is_complete.argtypes = [C.c_char_p, C.c_size_t]
        L.pgo_json_allowed_bytes.argtypes = [C.c_char_p, C.c_size_t, u8p]
        _lib = L
    return _lib


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a, ty):
    return a.ctypes.data_as(C.POINTER(ty)) if a is not None else None


class Rng:
    """SplitMix64 stream of the reference (rng.rs:7-31)."""

    def __init__(self, seed: int):
        self._s = C.c_uint64(0)
        lib().pgo_rng_new(C.byref(self._s), C.c_uint64(seed))

    def next_u64(self) -> int:
        return lib().pgo_rng_next_u64(C.byref(self._s))

    def next_f64(self) -> float:
        return lib().pgo_rng_next_f64(C.byref(self._s))

    def next_f32(self) -> float:
        return lib().pgo_rng_next_f32(C.byref(self._s))


def argmax(xs) -> int:
    xs = _f32(xs)
    return lib().pgo_argmax(_ptr(xs, C.c_float), xs.size)


def log_softmax(xs):
    xs = _f32(xs)
    out = np.empty_like(xs)
    lib().pgo_log_softmax(_ptr(xs, C.c_float), xs.size, _ptr(out, C.c_float))
    return out


def temperature_softmax(xs, temp):
    xs = _f32(xs).copy()
    lib().pgo_temperature_softmax(_ptr(xs, C.c_float), xs.size, temp)
    return xs


def apply_top_k(xs, k):
    xs = _f32(xs).copy()
    lib().pgo_apply_top_k(_ptr(xs, C.c_float), xs.size, k)
    return xs


def apply_top_p(xs, p):
    xs = _f32(xs).copy()
    lib().pgo_apply_top_p(_ptr(xs, C.c_float), xs.size, p)
    return xs


def sample_categorical(probs, u):
    probs = _f32(probs)
    drew = C.c_int(0)
    tok = lib().pgo_sample_categorical(_ptr(probs, C.c_float), probs.size, u, C.byref(drew))
    return tok, bool(drew.value)


def sample(logits, temperature=0.0, top_k=0, top_p=1.0, u=0.0):
    logits = _f32(logits)
    drew = C.c_int(0)
    tok = lib().pgo_sample(_ptr(logits, C.c_float), logits.size, temperature, top_k, top_p, u, C.byref(drew))
    return tok, bool(drew.value)


class Sampler:
    """Mirror of `pagoda::Sampler` (sampler.rs:11-55): one RNG stream, one draw per stochastic call."""

    def __init__(self, seed: int):
        self.rng = Rng(seed)

    def seed(self, seed: int):
        self.rng = Rng(seed)

    def sample(self, logits, temperature=0.0, top_k=0, top_p=1.0) -> int:
        if temperature < 1e-5:
            return argmax(logits)
        probs = apply_top_p(apply_top_k(temperature_softmax(logits, temperature), top_k), top_p)
        return self.sample_categorical(probs)

    def sample_categorical(self, probs) -> int:
        probs = _f32(probs)
        # the reference only draws when total > EPS (sampler.rs:42-46)
        tok, drew = sample_categorical(probs, 0.0)
        if not drew:
            return tok
        return sample_categorical(probs, self.rng.next_f32())[0]


def apply_penalties(logits, output, freq=0.0, pres=0.0):
    logits = _f32(logits).copy()
    out = np.ascontiguousarray(output, dtype=np.uint32)
    lib().pgo_apply_penalties(_ptr(logits, C.c_float), logits.size, _ptr(out, C.c_uint32), out.size, freq, pres)
    return logits


def apply_repetition(logits, output, rep):
    logits = _f32(logits).copy()
    out = np.ascontiguousarray(output, dtype=np.uint32)
    lib().pgo_apply_repetition(_ptr(logits, C.c_float), logits.size, _ptr(out, C.c_uint32), out.size, rep)
    return logits


def mask_logits_bytes(allowed: bytes, logits):
    logits = _f32(logits).copy()
    a = np.frombuffer(bytes(allowed), dtype=np.uint8).copy()
    lib().pgo_mask_logits_bytes(_ptr(a, C.c_uint8), a.size, _ptr(logits, C.c_float), logits.size)
    return logits


def mask_logits_bits(words, logits):
    logits = _f32(logits).copy()
    w = np.ascontiguousarray(words, dtype=np.uint32)
    lib().pgo_mask_logits_bits(_ptr(w, C.c_uint32), _ptr(logits, C.c_float), logits.size)
    return logits


def bf16_to_f32(bits):
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(bits.shape, dtype=np.float32)
    lib().pgo_bf16_to_f32(_ptr(bits, C.c_uint16), _ptr(out, C.c_float), bits.size)
    return out


def _row_params(temperature=0.0, top_k=0, top_p=1.0, freq=0.0, pres=0.0, rep=1.0, history=None,
                mask_words=None, dead=False, complete=False, eos_id=-1, uniform=0.0):
    p = RowParams()
    p.temperature, p.top_p, p.top_k = temperature, top_p, top_k
    p.freq, p.pres, p.rep = freq, pres, rep
    hist = np.ascontiguousarray(history if history is not None else [], dtype=np.uint32)
    p.history, p.n_history = _ptr(hist, C.c_uint32), hist.size
    mw = np.ascontiguousarray(mask_words, dtype=np.uint32) if mask_words is not None else None
    p.mask_words = _ptr(mw, C.c_uint32)
    p.grammar_dead, p.grammar_complete, p.eos_id, p.uniform = int(dead), int(complete), eos_id, uniform
    return p, (hist, mw)


def sample_row(logits, want_probs=False, **params):
    logits = _f32(logits)
    n = logits.size
    p, _keep = _row_params(**params)
    out = RowOut()
    work = np.empty(2 * n, dtype=np.float32)
    probs = np.empty(n, dtype=np.float32) if want_probs else None
    lib().pgo_sample_row(_ptr(logits, C.c_float), n, C.byref(p), C.byref(out), _ptr(work, C.c_float),
                         _ptr(probs, C.c_float))
    return (out, probs) if want_probs else out


def sample_batch(logits, temperature=None, top_k=None, top_p=None, freq=None, pres=None, rep=None,
                 hist_offsets=None, hist_ids=None, mask_table=None, mask_state=None, state_flags=None,
                 eos_id=-1, uniform=None, n_threads=1):
    """Run the whole chain on a [rows, vocab] float32 array. `mask_table` is [states, words];
    `mask_state[r]` < 0 means no grammar on row r. Returns a structured array (ROW_OUT_DTYPE)."""
    logits = _f32(logits)
    rows, vocab = logits.shape
    b = Batch()
    keep = []

    def arr(a, dt, ty):
        if a is None:
            return None
        a = np.ascontiguousarray(a, dtype=dt)
        keep.append(a)
        return _ptr(a, ty)

    b.logits, b.rows, b.vocab, b.row_stride = _ptr(logits, C.c_float), rows, vocab, vocab
    b.temperature, b.top_p = arr(temperature, np.float32, C.c_float), arr(top_p, np.float32, C.c_float)
    b.top_k = arr(top_k, np.uint32, C.c_uint32)
    b.freq, b.pres, b.rep = (arr(freq, np.float32, C.c_float), arr(pres, np.float32, C.c_float),
                             arr(rep, np.float32, C.c_float))
    b.hist_offsets, b.hist_ids = arr(hist_offsets, np.uint32, C.c_uint32), arr(hist_ids, np.uint32, C.c_uint32)
    if mask_table is not None and mask_state is not None:
        table = np.ascontiguousarray(mask_table, dtype=np.uint32)
        keep.append(table)
        ptrs = (C.POINTER(C.c_uint32) * rows)()
        flags = np.zeros(rows, dtype=np.uint8)
        for r in range(rows):
            s = int(mask_state[r])
            if s >= 0:
                ptrs[r] = table[s].ctypes.data_as(C.POINTER(C.c_uint32))
                if state_flags is not None:
                    flags[r] = state_flags[s]
        keep.append(ptrs)
        keep.append(flags)
        b.mask_rows = ptrs
        b.row_flags = _ptr(flags, C.c_uint8)
    b.eos_id = eos_id
    b.uniform = arr(uniform, np.float32, C.c_float)
    out = np.zeros(rows, dtype=ROW_OUT_DTYPE)
    lib().pgo_sample_batch(C.byref(b), out.ctypes.data, n_threads)
    return out


def tp_sample_row(logits, n_shards, cand, temperature, top_p, u, **chain):
    """`chain`: top_k, freq, pres, rep, history, mask_words (whole row), dead, complete, eos_id."""
    logits = _f32(logits)
    p, _keep = _row_params(temperature=temperature, top_p=top_p, uniform=u, **chain)
    out = TpOut()
    lib().pgo_tp_sample_row(_ptr(logits, C.c_float), logits.size, n_shards, cand, C.byref(p), C.byref(out))
    return out


def draft_accept(row_argmax, draft):
    a = np.ascontiguousarray(row_argmax, dtype=np.uint32)
    d = np.ascontiguousarray(draft, dtype=np.uint32)
    nxt = C.c_uint32(0)
    n = lib().pgo_draft_accept(_ptr(a, C.c_uint32), _ptr(d, C.c_uint32), a.size, C.byref(nxt))
    return n, nxt.value


class Regex:
    """`ByteRegex` of the reference (grammar.rs:458-575)."""

    def __init__(self, pattern: str):
        err = C.create_string_buffer(256)
        self._h = lib().pgo_regex_new(pattern.encode("latin-1"), err, 256)
        if not self._h:
            raise ValueError(err.value.decode())

    def __del__(self):
        if getattr(self, "_h", None):
            lib().pgo_regex_free(self._h)
            self._h = None

    def is_complete(self, text: bytes) -> bool:
        return bool(lib().pgo_regex_is_complete(self._h, text, len(text)))

    def allowed_bytes(self, text: bytes):
        out = (C.c_uint8 * 256)()
        n = lib().pgo_regex_allowed_bytes(self._h, text, len(text), out)
        return None if n < 0 else bytes(out[:n])


class Json:
    """`Grammar::Json` of the reference (grammar.rs:582-1016)."""

    @staticmethod
    def is_complete(text: bytes) -> bool:
        return bool(lib().pgo_json_is_complete(text, len(text)))

    @staticmethod
    def allowed_bytes(text: bytes):
        out = (C.c_uint8 * 256)()
        n = lib().pgo_json_allowed_bytes(text, len(text), out)
        return None if n < 0 else bytes(out[:n])
