"""ctypes binding of include/pagoda_sampler.h.

Host arrays (numpy) go through the host-memory side of the ABI; CUDA tensors (torch) are passed
as raw device pointers.  torch is only used for device memory and streams.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

PGS_F32, PGS_BF16 = 0, 1
MEM_DEVICE, MEM_HOST = 0, 1
ROW_OK, ROW_NONFINITE, ROW_DEAD, ROW_EMPTY, ROW_BAD_PARAM = 0, 1, 2, 3, 4

EXPORTS = ["pgs_create", "pgs_destroy", "pgs_last_error", "pgs_mask_table_upload", "pgs_mask_table_free",
           "pgs_sample_batch", "pgs_sample_batch_async", "pgs_get_counters", "pgs_stream", "pgs_set_exact",
           "pgs_sample_batch_static", "pgs_static_last_error",
           "pgs_grammar_regex", "pgs_grammar_json", "pgs_grammar_free", "pgs_grammar_n_states",
           "pgs_grammar_build_table", "pgs_grammar_state_new", "pgs_grammar_state_reset", "pgs_grammar_state_free",
           "pgs_grammar_advance", "pgs_grammar_mask_state", "pgs_grammar_state_info",
           "pgs_log_softmax", "pgs_tp_record_bytes", "pgs_tp_partial", "pgs_tp_merge", "pgs_tp_partial_push",
           "pgs_tp_merge_wait", "pgs_set_wait_limit", "pgs_tp_exchange_status", "pgs_debug_read_profile", "pgs_peer_alloc", "pgs_peer_open", "pgs_peer_close", "pgs_peer_free", "pgs_draft_accept"]


class SamplerError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"pgs error {code}: {msg}")
        self.code = code


class BatchDesc(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("rows", C.c_uint32), ("vocab", C.c_uint32), ("logits_dtype", C.c_uint32),
        ("row_stride", C.c_uint64), ("logits", C.c_void_p), ("logits_mem", C.c_uint32), ("aux_mem", C.c_uint32),
        ("temperature", C.c_void_p), ("top_k", C.c_void_p), ("top_p", C.c_void_p),
        ("frequency_penalty", C.c_void_p), ("presence_penalty", C.c_void_p), ("repetition_penalty", C.c_void_p),
        ("hist_offsets", C.c_void_p), ("hist_ids", C.c_void_p),
        ("mask_table", C.c_void_p), ("mask_state", C.c_void_p),
        ("eos_token_id", C.c_int32), ("reserved0", C.c_uint32), ("uniform", C.c_void_p),
        ("token", C.c_void_p), ("status", C.c_void_p), ("drew", C.c_void_p),
        ("argmax", C.c_void_p), ("row_max", C.c_void_p), ("sumexp", C.c_void_p), ("total", C.c_void_p),
        ("n_kept", C.c_void_p), ("dump_cap", C.c_uint32), ("reserved1", C.c_uint32),
        ("dump_ids", C.c_void_p), ("dump_probs", C.c_void_p),
    ]


class TpDesc(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("rows", C.c_uint32), ("vocab", C.c_uint32), ("n_shards", C.c_uint32),
                ("shard_rank", C.c_uint32), ("cand", C.c_uint32), ("row_stride", C.c_uint64),
                ("logits", C.c_void_p), ("temperature", C.c_void_p), ("top_p", C.c_void_p), ("uniform", C.c_void_p),
                ("top_k", C.c_void_p),
                ("frequency_penalty", C.c_void_p), ("presence_penalty", C.c_void_p), ("repetition_penalty", C.c_void_p),
                ("hist_offsets", C.c_void_p), ("hist_ids", C.c_void_p),
                ("mask_table", C.c_void_p), ("mask_state", C.c_void_p),
                ("eos_token_id", C.c_int32), ("reserved0", C.c_int32)]


class TpOut(C.Structure):
    _fields_ = [("token", C.c_void_p), ("status", C.c_void_p), ("drew", C.c_void_p), ("argmax", C.c_void_p),
                ("gmax", C.c_void_p), ("gsum", C.c_void_p), ("total", C.c_void_p), ("n_kept", C.c_void_p)]


class Counters(C.Structure):
    _fields_ = [("calls", C.c_uint64), ("rows", C.c_uint64), ("rows_faulted", C.c_uint64), ("bytes", C.c_uint64),
                ("kernel_launches", C.c_uint64)]


def lib_path() -> str:
    return os.path.join(_HERE, "libpagoda_sampler.so")


_lib = None


def load_library():
    """dlopen the built library and declare its signatures. Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        raise SamplerError(-2, f"{path} is missing: build it with `python -m pagoda_b200.build` "
                               "(there is no CPU fallback)")
    L = C.CDLL(path)
    L.pgs_create.argtypes = [C.c_int, C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(C.c_void_p)]
    L.pgs_destroy.argtypes = [C.c_void_p]
    L.pgs_last_error.restype = C.c_char_p
    L.pgs_last_error.argtypes = [C.c_void_p]
    L.pgs_mask_table_upload.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p,
                                        C.POINTER(C.c_int32)]
    L.pgs_mask_table_free.argtypes = [C.c_void_p, C.c_int32]
    L.pgs_sample_batch.argtypes = [C.c_void_p, C.POINTER(BatchDesc)]
    L.pgs_sample_batch_async.argtypes = [C.c_void_p, C.POINTER(BatchDesc), C.c_void_p]
    L.pgs_get_counters.argtypes = [C.c_void_p, C.POINTER(Counters)]
    L.pgs_set_exact.argtypes = [C.c_void_p, C.c_int]
    L.pgs_sample_batch_static.argtypes = [C.c_int, C.POINTER(BatchDesc), C.c_void_p]
    L.pgs_static_last_error.restype = C.c_char_p
    L.pgs_grammar_regex.argtypes = [C.c_char_p, C.POINTER(C.c_void_p), C.c_char_p, C.c_size_t]
    L.pgs_grammar_json.argtypes = [C.POINTER(C.c_void_p)]
    L.pgs_grammar_free.argtypes = [C.c_void_p]
    L.pgs_grammar_free.restype = None
    L.pgs_grammar_n_states.argtypes = [C.c_void_p]
    L.pgs_grammar_n_states.restype = C.c_uint32
    L.pgs_grammar_build_table.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p]
    L.pgs_grammar_state_new.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
    L.pgs_grammar_state_reset.argtypes = [C.c_void_p, C.c_void_p]
    L.pgs_grammar_state_free.argtypes = [C.c_void_p]
    L.pgs_grammar_state_free.restype = None
    L.pgs_grammar_advance.argtypes = [C.c_void_p, C.c_void_p, C.c_char_p, C.c_size_t]
    L.pgs_grammar_mask_state.argtypes = [C.c_void_p, C.c_void_p]
    L.pgs_grammar_mask_state.restype = C.c_uint32
    L.pgs_grammar_state_info.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int)]
    L.pgs_log_softmax.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint64, C.c_void_p, C.c_void_p,
                                  C.c_void_p, C.c_void_p, C.c_void_p]
    L.pgs_tp_record_bytes.restype = C.c_size_t
    L.pgs_tp_record_bytes.argtypes = [C.c_uint32]
    L.pgs_tp_partial.argtypes = [C.c_void_p, C.POINTER(TpDesc), C.c_void_p, C.c_void_p]
    L.pgs_tp_merge.argtypes = [C.c_void_p, C.POINTER(TpDesc), C.c_void_p, C.POINTER(TpOut), C.c_void_p]
    L.pgs_tp_partial_push.argtypes = [C.c_void_p, C.POINTER(TpDesc), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                      C.c_uint32, C.c_void_p]
    L.pgs_debug_read_profile.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32]
    L.pgs_peer_alloc.argtypes = [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p), C.c_char_p]
    L.pgs_peer_open.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_void_p)]
    L.pgs_peer_close.argtypes = [C.c_void_p, C.c_void_p]
    L.pgs_peer_free.argtypes = [C.c_void_p, C.c_void_p]
    L.pgs_set_wait_limit.argtypes = [C.c_void_p, C.c_uint32]
    L.pgs_tp_exchange_status.argtypes = [C.c_void_p]
    L.pgs_tp_merge_wait.argtypes = [C.c_void_p, C.POINTER(TpDesc), C.c_void_p, C.c_void_p, C.c_uint32,
                                    C.POINTER(TpOut), C.c_void_p]
    L.pgs_draft_accept.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p,
                                   C.c_void_p, C.c_void_p]
    L.pgs_stream.restype = C.c_void_p
    L.pgs_stream.argtypes = [C.c_void_p]
    _lib = L
    return L


def _is_torch(x) -> bool:
    return x is not None and type(x).__module__.startswith("torch")


@dataclass
class BatchResult:
    token: np.ndarray
    status: np.ndarray
    drew: np.ndarray
    argmax: Optional[np.ndarray] = None
    row_max: Optional[np.ndarray] = None
    sumexp: Optional[np.ndarray] = None
    total: Optional[np.ndarray] = None
    n_kept: Optional[np.ndarray] = None
    dump_ids: Optional[np.ndarray] = None
    dump_probs: Optional[np.ndarray] = None

    def kept(self, row: int):
        n = min(int(self.n_kept[row]), self.dump_ids.shape[1])
        return self.dump_ids[row, :n], self.dump_probs[row, :n]


def sample_batch_static(device: int, desc: "BatchDesc", stream_ptr: Optional[int] = None):
    """pgs_sample_batch_static: the allocation-free entry point (fixed in-library working storage,
    no handle).  `desc` is a device-resident descriptor as built by Sampler.make_device_desc."""
    L = load_library()
    rc = L.pgs_sample_batch_static(device, C.byref(desc), Sampler._stream(stream_ptr))
    if rc != 0:
        raise SamplerError(rc, L.pgs_static_last_error().decode())


class GrammarState:
    """Per-sequence host state of a grammar: advanced by the emitted bytes, read as a table state."""

    def __init__(self, grammar: "Grammar"):
        self.g = grammar
        self._s = C.c_void_p()
        rc = load_library().pgs_grammar_state_new(grammar._g, C.byref(self._s))
        if rc != 0:
            raise SamplerError(rc, "pgs_grammar_state_new failed")

    def __del__(self):
        if getattr(self, "_s", None):
            load_library().pgs_grammar_state_free(self._s)
            self._s = None

    def reset(self):
        load_library().pgs_grammar_state_reset(self.g._g, self._s)

    def advance(self, data: bytes):
        load_library().pgs_grammar_advance(self.g._g, self._s, data, len(data))

    @property
    def mask_state(self) -> int:
        return load_library().pgs_grammar_mask_state(self.g._g, self._s)

    def allowed_bytes(self):
        """`Grammar::allowed_bytes` of the reference for the bytes fed so far: None when dead."""
        allowed, complete, dead = self.g.state_info(self.mask_state)
        return None if dead else allowed

    def is_complete(self) -> bool:
        return self.g.state_info(self.mask_state)[1]


class Grammar:
    """A tabulated grammar (mirror of `pagoda::Grammar`: `Grammar.regex(pattern)`, `Grammar.json()`)."""

    def __init__(self, handle, name):
        self._g, self.name = handle, name

    @classmethod
    def regex(cls, pattern: str) -> "Grammar":
        g = C.c_void_p()
        err = C.create_string_buffer(256)
        rc = load_library().pgs_grammar_regex(pattern.encode("latin-1"), C.byref(g), err, 256)
        if rc != 0:
            raise ValueError(err.value.decode())
        return cls(g, "regex")

    @classmethod
    def json(cls) -> "Grammar":
        g = C.c_void_p()
        load_library().pgs_grammar_json(C.byref(g))
        return cls(g, "json")

    def __del__(self):
        if getattr(self, "_g", None):
            load_library().pgs_grammar_free(self._g)
            self._g = None

    @property
    def n_states(self) -> int:
        return load_library().pgs_grammar_n_states(self._g)

    def state_info(self, state: int):
        a = (C.c_uint8 * 256)()
        c, d = C.c_int(0), C.c_int(0)
        rc = load_library().pgs_grammar_state_info(self._g, state, a, C.byref(c), C.byref(d))
        if rc != 0:
            raise SamplerError(rc, "bad grammar state")
        return bytes(b for b in range(256) if a[b]), bool(c.value), bool(d.value)

    def build_table(self, vocab: int, first_byte_id: int = 3):
        """(words [n_states, ceil(vocab/32)] uint32, flags [n_states] uint8) for upload_mask_table."""
        n = self.n_states
        words = np.zeros((n, (vocab + 31) // 32), dtype=np.uint32)
        flags = np.zeros(n, dtype=np.uint8)
        rc = load_library().pgs_grammar_build_table(self._g, vocab, first_byte_id, words.ctypes.data, flags.ctypes.data)
        if rc != 0:
            raise SamplerError(rc, "pgs_grammar_build_table failed")
        return words, flags

    def new_state(self) -> GrammarState:
        return GrammarState(self)


class Sampler:
    """One device-side sampler backend (a `pgs_handle`)."""

    def __init__(self, device: int = 0, max_rows: int = 256, max_vocab: int = 262144, max_history: int = 4096):
        self._lib = load_library()
        self._h = C.c_void_p()
        rc = self._lib.pgs_create(device, max_rows, max_vocab, max_history, C.byref(self._h))
        if rc != 0:
            raise SamplerError(rc, self._lib.pgs_last_error(None).decode())
        self.device = device
        self.max_rows, self.max_vocab, self.max_history = max_rows, max_vocab, max_history

    def close(self):
        if getattr(self, "_h", None):
            self._lib.pgs_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int):
        if rc != 0:
            raise SamplerError(rc, self._lib.pgs_last_error(self._h).decode())

    def set_exact(self, on: bool):
        """Route every row through the bit-exact general kernel (see pgs_set_exact)."""
        self._check(self._lib.pgs_set_exact(self._h, int(on)))

    @property
    def stream_ptr(self) -> int:
        return self._lib.pgs_stream(self._h)

    def counters(self) -> dict:
        c = Counters()
        self._check(self._lib.pgs_get_counters(self._h, C.byref(c)))
        return {k: getattr(c, k) for k, _ in Counters._fields_}

    def read_phase_timers(self, n_ctas: int = 1024):
        """Cycles per CTA and phase of the streaming row kernel since the last read ([n_ctas, 16] int64; needs
        PGS_PROFILE=1 in the environment when the sampler is created)."""
        out = np.zeros((n_ctas, 16), dtype=np.int64)
        self._check(self._lib.pgs_debug_read_profile(self._h, out.ctypes.data_as(C.c_void_p), C.c_uint32(n_ctas)))
        return out

    def upload_mask_table(self, words, state_flags=None) -> int:
        words = np.ascontiguousarray(words, dtype=np.uint32)
        assert words.ndim == 2
        flags = None if state_flags is None else np.ascontiguousarray(state_flags, dtype=np.uint8)
        tid = C.c_int32(-1)
        self._check(self._lib.pgs_mask_table_upload(
            self._h, words.shape[0], words.shape[1], words.ctypes.data,
            None if flags is None else flags.ctypes.data, C.byref(tid)))
        return tid.value

    def free_mask_table(self, table_id: int):
        self._check(self._lib.pgs_mask_table_free(self._h, table_id))

    # ------------------------------------------------------------------ host-resident batch
    def sample_batch(self, logits, temperature=None, top_k=None, top_p=None, frequency_penalty=None,
                     presence_penalty=None, repetition_penalty=None, hist_offsets=None, hist_ids=None,
                     mask_table=None, mask_state=None, eos_token_id=-1, uniform=None, diagnostics=False,
                     dump_cap=0, row_stride=None, vocab=None) -> BatchResult:
        """`logits`: numpy [rows, vocab] float32, or uint16 holding bf16 bit patterns; or a CUDA
        torch tensor (float32 / bfloat16), in which case only the per-row arrays are staged."""
        keep = []
        d = BatchDesc()
        d.struct_size = C.sizeof(BatchDesc)
        if _is_torch(logits):
            import torch
            assert logits.is_cuda and logits.dim() == 2 and logits.stride(1) == 1
            rows = logits.shape[0]
            d.vocab = logits.shape[1] if vocab is None else vocab
            d.row_stride = logits.stride(0)
            d.logits_dtype = PGS_BF16 if logits.dtype == torch.bfloat16 else PGS_F32
            assert logits.dtype in (torch.float32, torch.bfloat16)
            d.logits = logits.data_ptr()
            d.logits_mem = MEM_DEVICE
            keep.append(logits)
        else:
            logits = np.asarray(logits)
            assert logits.ndim == 2 and logits.dtype in (np.float32, np.uint16)
            if not logits.flags.c_contiguous and row_stride is None:
                logits = np.ascontiguousarray(logits)
            rows = logits.shape[0]
            d.vocab = logits.shape[1] if vocab is None else vocab
            d.row_stride = logits.shape[1] if row_stride is None else row_stride
            d.logits_dtype = PGS_F32 if logits.dtype == np.float32 else PGS_BF16
            d.logits = logits.ctypes.data
            d.logits_mem = MEM_HOST
            keep.append(logits)
        d.rows = rows
        d.aux_mem = MEM_HOST
        d.eos_token_id = eos_token_id

        def arr(x, dt, n=rows):
            if x is None:
                return None
            a = np.ascontiguousarray(np.broadcast_to(np.asarray(x, dtype=dt), (n,)) if np.ndim(x) == 0 else x,
                                     dtype=dt)
            assert a.size == n, (a.size, n)
            keep.append(a)
            return a.ctypes.data

        d.temperature = arr(temperature, np.float32)
        d.top_k = arr(top_k, np.uint32)
        d.top_p = arr(top_p, np.float32)
        d.frequency_penalty = arr(frequency_penalty, np.float32)
        d.presence_penalty = arr(presence_penalty, np.float32)
        d.repetition_penalty = arr(repetition_penalty, np.float32)
        if hist_offsets is not None:
            ho = np.ascontiguousarray(hist_offsets, dtype=np.uint32)
            hi = np.ascontiguousarray(hist_ids if hist_ids is not None else [], dtype=np.uint32)
            assert ho.size == rows + 1
            keep += [ho, hi]
            d.hist_offsets, d.hist_ids = ho.ctypes.data, hi.ctypes.data
        d.mask_table = arr(mask_table, np.int32)
        d.mask_state = arr(mask_state, np.int32)
        d.uniform = arr(uniform, np.float32)
        res = BatchResult(np.zeros(rows, np.uint32), np.full(rows, -1, np.int32), np.zeros(rows, np.uint8))
        d.token, d.status, d.drew = res.token.ctypes.data, res.status.ctypes.data, res.drew.ctypes.data
        if diagnostics or dump_cap:
            res.argmax = np.zeros(rows, np.uint32)
            res.row_max = np.zeros(rows, np.float32)
            res.sumexp = np.zeros(rows, np.float32)
            res.total = np.zeros(rows, np.float32)
            res.n_kept = np.zeros(rows, np.uint32)
            d.argmax, d.row_max, d.sumexp = res.argmax.ctypes.data, res.row_max.ctypes.data, res.sumexp.ctypes.data
            d.total, d.n_kept = res.total.ctypes.data, res.n_kept.ctypes.data
        if dump_cap:
            res.dump_ids = np.zeros((rows, dump_cap), np.uint32)
            res.dump_probs = np.zeros((rows, dump_cap), np.float32)
            d.dump_cap = dump_cap
            d.dump_ids, d.dump_probs = res.dump_ids.ctypes.data, res.dump_probs.ctypes.data
        self._check(self._lib.pgs_sample_batch(self._h, C.byref(d)))
        return res

    # ---------------------------------------------------------------- device-resident batch
    def make_device_desc(self, logits, token, status, temperature=None, top_k=None, top_p=None,
                         frequency_penalty=None, presence_penalty=None, repetition_penalty=None,
                         hist_offsets=None, hist_ids=None, mask_table=None, mask_state=None, eos_token_id=-1,
                         uniform=None, drew=None, argmax=None, row_max=None, sumexp=None, total=None,
                         n_kept=None):
        """Build a descriptor whose every array is a CUDA torch tensor (kept alive by the returned
        object); launch it with `launch_device`."""
        import torch
        d = BatchDesc()
        d.struct_size = C.sizeof(BatchDesc)
        d.rows, d.vocab = logits.shape
        d.row_stride = logits.stride(0)
        d.logits_dtype = PGS_BF16 if logits.dtype == torch.bfloat16 else PGS_F32
        d.logits, d.logits_mem, d.aux_mem = logits.data_ptr(), MEM_DEVICE, MEM_DEVICE
        d.eos_token_id = eos_token_id
        keep = [logits]

        def p(t, dt):
            if t is None:
                return None
            assert t.is_cuda and t.is_contiguous() and t.dtype == dt, (t.dtype, dt)
            keep.append(t)
            return t.data_ptr()

        d.temperature, d.top_k, d.top_p = p(temperature, torch.float32), p(top_k, torch.int32), p(top_p, torch.float32)
        d.frequency_penalty, d.presence_penalty = p(frequency_penalty, torch.float32), p(presence_penalty, torch.float32)
        d.repetition_penalty = p(repetition_penalty, torch.float32)
        d.hist_offsets, d.hist_ids = p(hist_offsets, torch.int32), p(hist_ids, torch.int32)
        d.mask_table, d.mask_state = p(mask_table, torch.int32), p(mask_state, torch.int32)
        d.uniform = p(uniform, torch.float32)
        d.token, d.status, d.drew = p(token, torch.int32), p(status, torch.int32), p(drew, torch.uint8)
        d.argmax, d.row_max, d.sumexp = p(argmax, torch.int32), p(row_max, torch.float32), p(sumexp, torch.float32)
        d.total, d.n_kept = p(total, torch.float32), p(n_kept, torch.int32)
        d._keep = keep
        return d

    @staticmethod
    def _stream(stream_ptr):
        """None = the handle's own stream.  torch reports its default stream as 0, which the C ABI
        reads as "the handle's stream", so 0 is translated to CUDA's legacy-default-stream handle."""
        if stream_ptr is None:
            return None
        return stream_ptr if stream_ptr else 1   # cudaStreamLegacy

    def launch_device(self, desc, stream_ptr: Optional[int] = None):
        """Enqueue one step without waiting (pgs_sample_batch_async)."""
        self._check(self._lib.pgs_sample_batch_async(self._h, C.byref(desc), self._stream(stream_ptr)))

    # ------------------------------------------------------------ vocabulary-sharded sampling
    def tp_record_bytes(self, cand: int) -> int:
        return self._lib.pgs_tp_record_bytes(cand)

    def _tp_desc(self, rows, vocab, n_shards, rank, cand, logits=None, temperature=None, top_p=None, uniform=None,
                 top_k=None, frequency_penalty=None, presence_penalty=None, repetition_penalty=None,
                 hist_offsets=None, hist_ids=None, mask_table=None, mask_state=None, eos_token_id=-1):
        """Per-row arrays are CUDA tensors (float32 / int32) or None."""
        d = TpDesc()
        self._tp_keep = (top_k, frequency_penalty, presence_penalty, repetition_penalty, hist_offsets, hist_ids,
                         mask_table, mask_state)
        ptr = lambda t: None if t is None else t.data_ptr()
        d.top_k, d.frequency_penalty, d.presence_penalty = ptr(top_k), ptr(frequency_penalty), ptr(presence_penalty)
        d.repetition_penalty, d.hist_offsets, d.hist_ids = ptr(repetition_penalty), ptr(hist_offsets), ptr(hist_ids)
        d.mask_table, d.mask_state, d.eos_token_id = ptr(mask_table), ptr(mask_state), int(eos_token_id)
        d.struct_size = C.sizeof(TpDesc)
        d.rows, d.vocab, d.n_shards, d.shard_rank, d.cand = rows, vocab, n_shards, rank, cand
        if logits is not None:
            assert logits.is_cuda and logits.stride(1) == 1
            d.row_stride, d.logits = logits.stride(0), logits.data_ptr()
        else:
            d.row_stride = vocab // n_shards
        d.temperature = None if temperature is None else temperature.data_ptr()
        d.top_p = None if top_p is None else top_p.data_ptr()
        d.uniform = None if uniform is None else uniform.data_ptr()
        return d

    def tp_partial(self, shard_logits, vocab, n_shards, rank, cand, temperature=None, records=None, stream_ptr=None,
                   **chain):
        """Emit this rank's per-row records (uint8 CUDA tensor [rows, record_bytes]) for its column
        shard `shard_logits` [rows, vocab // n_shards] (float32, CUDA).  `chain`: the penalty / history /
        grammar arguments of _tp_desc (history ids and eos_token_id are global ids, mask tables hold this
        shard's bits)."""
        import torch
        rows = shard_logits.shape[0]
        if records is None:
            records = torch.empty((rows, self.tp_record_bytes(cand)), dtype=torch.uint8, device=shard_logits.device)
        d = self._tp_desc(rows, vocab, n_shards, rank, cand, shard_logits, temperature, **chain)
        self._check(self._lib.pgs_tp_partial(self._h, C.byref(d), records.data_ptr(), self._stream(stream_ptr)))
        return records

    @staticmethod
    def tp_outputs(rows, dev):
        """Output tensors of tp_merge / tp_merge_wait (pass them back in as `out` to reuse them)."""
        import torch
        return dict(token=torch.zeros(rows, dtype=torch.int32, device=dev),
                    status=torch.full((rows,), -1, dtype=torch.int32, device=dev),
                    drew=torch.zeros(rows, dtype=torch.uint8, device=dev),
                    argmax=torch.zeros(rows, dtype=torch.int32, device=dev),
                    gmax=torch.zeros(rows, dtype=torch.float32, device=dev),
                    gsum=torch.zeros(rows, dtype=torch.float32, device=dev),
                    total=torch.zeros(rows, dtype=torch.float32, device=dev),
                    n_kept=torch.zeros(rows, dtype=torch.int32, device=dev))

    def tp_merge(self, records_all, vocab, n_shards, rank, cand, temperature=None, top_p=None, uniform=None,
                 stream_ptr=None, top_k=None, out=None):
        """Merge the all-gathered records [n_shards, rows, record_bytes] into tokens; returns a dict of
        CUDA tensors (token, status, drew, argmax, gmax, gsum, total, n_kept)."""
        import torch
        rows = records_all.shape[1]
        dev = records_all.device
        out = self.tp_outputs(rows, dev) if out is None else out
        o = TpOut(**{k: v.data_ptr() for k, v in out.items()})
        d = self._tp_desc(rows, vocab, n_shards, rank, cand, None, temperature, top_p, uniform, top_k=top_k)
        self._check(self._lib.pgs_tp_merge(self._h, C.byref(d), records_all.data_ptr(), C.byref(o),
                                           self._stream(stream_ptr)))
        return out

    def peer_alloc(self, nbytes: int):
        """Zeroed device memory that peers can map: -> (device address, 64-byte IPC handle)."""
        ptr = C.c_void_p()
        handle = C.create_string_buffer(64)
        self._check(self._lib.pgs_peer_alloc(self._h, nbytes, C.byref(ptr), handle))
        return int(ptr.value), handle.raw

    def peer_open(self, ipc_handle: bytes) -> int:
        """Map a peer's buffer for this sampler's device: -> device address."""
        ptr = C.c_void_p()
        self._check(self._lib.pgs_peer_open(self._h, C.create_string_buffer(ipc_handle, 64), C.byref(ptr)))
        return int(ptr.value)

    def peer_close(self, addr: int):
        self._check(self._lib.pgs_peer_close(self._h, C.c_void_p(addr)))

    def peer_free(self, addr: int):
        self._check(self._lib.pgs_peer_free(self._h, C.c_void_p(addr)))

    def tp_partial_push(self, shard_logits, vocab, n_shards, rank, cand, peer_record_ptrs, peer_flag_ptrs, epoch,
                        temperature=None, stream_ptr=None, **chain):
        """Emit this rank's records straight into every rank's gather buffer (peer stores) and raise this
        shard's flag there.  peer_record_ptrs / peer_flag_ptrs: device addresses (ints), one per rank, of the
        [n_shards, rows, record_bytes] gather buffers and the [n_shards] uint32 flag arrays of this epoch."""
        rows = shard_logits.shape[0]
        d = self._tp_desc(rows, vocab, n_shards, rank, cand, shard_logits, temperature, **chain)
        recs = (C.c_void_p * n_shards)(*[int(p) for p in peer_record_ptrs])
        flags = (C.c_void_p * n_shards)(*[int(p) for p in peer_flag_ptrs])
        self._check(self._lib.pgs_tp_partial_push(self._h, C.byref(d), recs, flags, C.c_uint32(epoch),
                                                  self._stream(stream_ptr)))

    def set_wait_limit(self, polls: int):
        """Bound of tp_merge_wait's device-side wait, in polls of about half a microsecond."""
        self._check(self._lib.pgs_set_wait_limit(self._h, C.c_uint32(polls)))

    def tp_exchange_status(self):
        """Raises SamplerError (code -5) when rows gave up waiting for a shard since the last call."""
        self._check(self._lib.pgs_tp_exchange_status(self._h))

    def tp_merge_wait(self, records_all, flags, epoch, vocab, n_shards, rank, cand, temperature=None, top_p=None,
                      uniform=None, stream_ptr=None, top_k=None, out=None):
        """tp_merge preceded, on the device, by a bounded wait until all n_shards flags of this rank have
        reached `epoch`.  records_all [n_shards, rows, record_bytes] uint8, flags [n_shards] int32/uint32."""
        import torch
        rows = records_all.shape[1]
        dev = records_all.device
        out = self.tp_outputs(rows, dev) if out is None else out
        o = TpOut(**{k: v.data_ptr() for k, v in out.items()})
        d = self._tp_desc(rows, vocab, n_shards, rank, cand, None, temperature, top_p, uniform, top_k=top_k)
        self._check(self._lib.pgs_tp_merge_wait(self._h, C.byref(d), C.c_void_p(records_all.data_ptr()),
                                                C.c_void_p(flags.data_ptr()), C.c_uint32(epoch), C.byref(o),
                                                self._stream(stream_ptr)))
        return out

    def draft_accept(self, row_argmax, draft, stream_ptr=None, out=None):
        """row_argmax, draft: int32 CUDA tensors [sequences, positions] -> (accepted, next); `out`: a pair of
        int32 tensors [sequences] to write into instead of new ones."""
        import torch
        seqs, pos = row_argmax.shape
        if out is None:
            out = (torch.zeros(seqs, dtype=torch.int32, device=row_argmax.device),
                   torch.zeros(seqs, dtype=torch.int32, device=row_argmax.device))
        acc, nxt = out
        self._check(self._lib.pgs_draft_accept(self._h, row_argmax.contiguous().data_ptr(),
                                               draft.contiguous().data_ptr(), seqs, pos, acc.data_ptr(),
                                               nxt.data_ptr(), self._stream(stream_ptr)))
        return acc, nxt

    # ------------------------------------------------------------------------------ scoring
    def log_softmax(self, logits, ids=None, full=False, stream_ptr=None):
        """`sampler::log_softmax` on a CUDA float32 tensor [rows, vocab]; returns (gathered [rows] or
        None, full [rows, vocab] or None, status [rows])."""
        import torch
        rows, vocab = logits.shape
        dev = logits.device
        gathered = torch.empty(rows, dtype=torch.float32, device=dev) if ids is not None else None
        out_full = torch.empty((rows, vocab), dtype=torch.float32, device=dev) if full else None
        status = torch.zeros(rows, dtype=torch.int32, device=dev)
        self._check(self._lib.pgs_log_softmax(
            self._h, logits.data_ptr(), rows, vocab, logits.stride(0), None if ids is None else ids.data_ptr(),
            None if gathered is None else gathered.data_ptr(), None if out_full is None else out_full.data_ptr(),
            status.data_ptr(), self._stream(stream_ptr)))
        return gathered, out_full, status
