"""Seeded synthetic workloads for the sampler path.

There is no dataset behind this path: the reference publishes no sampler benchmark, so the
five benchmark configurations are described by shapes and distributions only.  Everything here
is generated from a stated seed with the reference's own SplitMix64 stream (rng.rs:10-30) used
counter-style, uniforms as `next_f64`, and normals by Box-Muller.  "N(0, s)" means standard
deviation s.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np

GAMMA = np.uint64(0x9E3779B97F4A7C15)


def splitmix_u64(seed: int, n: int, offset: int = 0) -> np.ndarray:
    """Draws offset .. offset+n-1 of `Rng::new(seed)` (rng.rs:10-21)."""
    with np.errstate(over="ignore"):
        j = np.arange(offset + 2, offset + n + 2, dtype=np.uint64)
        z = np.uint64(seed & 0xFFFFFFFFFFFFFFFF) + GAMMA * j
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def uniform_f64(seed: int, n: int, offset: int = 0) -> np.ndarray:
    """`next_f64` (rng.rs:24-26): 53 random bits scaled into [0, 1)."""
    return (splitmix_u64(seed, n, offset) >> np.uint64(11)).astype(np.float64) * (1.0 / (1 << 53))


def uniform_f32(seed: int, n: int, offset: int = 0) -> np.ndarray:
    """`next_f32` (rng.rs:28-30); may round up to exactly 1.0."""
    return uniform_f64(seed, n, offset).astype(np.float32)


def normal_f32(seed: int, n: int, std: float) -> np.ndarray:
    m = (n + 1) // 2
    u = uniform_f64(seed, 2 * m)
    r = np.sqrt(-2.0 * np.log1p(-u[:m]))
    th = 2.0 * np.pi * u[m:]
    out = np.concatenate([r * np.cos(th), r * np.sin(th)])[:n]
    return (out * std).astype(np.float32)


def randint(seed: int, n: int, lo: int, hi: int) -> np.ndarray:
    """Integers uniform in [lo, hi)."""
    return (lo + (uniform_f64(seed, n) * (hi - lo)).astype(np.int64)).clip(lo, hi - 1)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 bit patterns (uint16)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


@dataclass
class Workload:
    name: str
    logits: np.ndarray                       # [rows, vocab] float32, or uint16 (bf16 bits)
    temperature: np.ndarray
    top_k: np.ndarray
    top_p: np.ndarray
    frequency_penalty: np.ndarray
    presence_penalty: np.ndarray
    repetition_penalty: np.ndarray
    hist_offsets: Optional[np.ndarray]
    hist_ids: Optional[np.ndarray]
    uniform: np.ndarray
    mask_words: Optional[np.ndarray] = None   # [states, words]
    state_flags: Optional[np.ndarray] = None
    mask_state: Optional[np.ndarray] = None   # per row, -1 = none
    eos_token_id: int = -1
    extra: dict = field(default_factory=dict)

    @property
    def rows(self):
        return self.logits.shape[0]

    @property
    def vocab(self):
        return self.logits.shape[1]

    @property
    def is_bf16(self):
        return self.logits.dtype == np.uint16

    def logits_f32(self) -> np.ndarray:
        return bf16_bits_to_f32(self.logits).reshape(self.logits.shape) if self.is_bf16 else self.logits

    def head(self, n: int) -> "Workload":
        """The first n rows as a workload of their own."""
        import copy
        w = copy.copy(self)
        for k in ("logits", "temperature", "top_k", "top_p", "frequency_penalty", "presence_penalty",
                  "repetition_penalty", "uniform"):
            setattr(w, k, getattr(self, k)[:n])
        if self.hist_offsets is not None:
            w.hist_offsets = self.hist_offsets[:n + 1]
        if self.mask_state is not None:
            w.mask_state = self.mask_state[:n]
        return w

    def algorithmic_bytes(self) -> int:
        """Bytes the chain has to touch: every logit once, the bitmask of masked rows, the history
        ids, and 64 B of per-row parameters and results."""
        esz = 2 if self.is_bf16 else 4
        total = self.rows * (self.vocab * esz + 64)
        if self.hist_offsets is not None:
            total += 4 * int(self.hist_offsets[-1])
        if self.mask_state is not None:
            total += int((self.mask_state >= 0).sum()) * (self.vocab // 8)
        return total

    def sampler_kwargs(self, table_id: Optional[int] = None) -> dict:
        kw = dict(temperature=self.temperature, top_k=self.top_k, top_p=self.top_p,
                  frequency_penalty=self.frequency_penalty, presence_penalty=self.presence_penalty,
                  repetition_penalty=self.repetition_penalty, hist_offsets=self.hist_offsets,
                  hist_ids=self.hist_ids, uniform=self.uniform, eos_token_id=self.eos_token_id)
        if self.mask_state is not None and table_id is not None:
            kw["mask_table"] = np.where(self.mask_state >= 0, table_id, -1).astype(np.int32)
            kw["mask_state"] = self.mask_state.astype(np.int32)
        return kw

    def oracle_kwargs(self) -> dict:
        kw = dict(temperature=self.temperature, top_k=self.top_k, top_p=self.top_p, freq=self.frequency_penalty,
                  pres=self.presence_penalty, rep=self.repetition_penalty, hist_offsets=self.hist_offsets,
                  hist_ids=self.hist_ids, uniform=self.uniform, eos_id=self.eos_token_id)
        if self.mask_state is not None:
            kw.update(mask_table=self.mask_words, mask_state=self.mask_state, state_flags=self.state_flags)
        return kw


def _const(rows, v, dt=np.float32):
    return np.full(rows, v, dtype=dt)


def _history(seed, rows, per_row, vocab):
    ids = randint(seed, rows * per_row, 0, vocab).astype(np.uint32)
    return np.arange(rows + 1, dtype=np.uint32) * np.uint32(per_row), ids


def config1(seed=1, rows=1, vocab=151936) -> Workload:
    """Greedy argmax with repetition penalty 1.1 over a 112-id history, f32 logits N(0, 3)."""
    ho, hi = _history(seed + 1000, rows, 112, vocab)
    return Workload("config1_greedy_rep", normal_f32(seed, rows * vocab, 3.0).reshape(rows, vocab),
                    _const(rows, 0.0), _const(rows, 0, np.uint32), _const(rows, 1.0), _const(rows, 0.0),
                    _const(rows, 0.0), _const(rows, 1.1), ho, hi, _const(rows, 0.0))


def config2(seed=2, rows=64, vocab=151936) -> Workload:
    """Batched stochastic sampling: f32 N(0, 2) with 8 ids per row spiked +10, T 0.7, top-k 50,
    top-p 0.9, frequency 0.2 / presence 0.1 over 512-id histories."""
    x = normal_f32(seed, rows * vocab, 2.0).reshape(rows, vocab)
    spikes = randint(seed + 2000, rows * 8, 0, vocab).reshape(rows, 8)
    for r in range(rows):
        x[r, spikes[r]] += np.float32(10.0)
    ho, hi = _history(seed + 1000, rows, 512, vocab)
    return Workload("config2_topk_topp", x, _const(rows, 0.7), _const(rows, 50, np.uint32), _const(rows, 0.9),
                    _const(rows, 0.2), _const(rows, 0.1), _const(rows, 1.0), ho, hi,
                    uniform_f32(seed + 3000, rows))


def random_mask_table(seed, n_states, vocab, lo=0.01, hi=0.20) -> np.ndarray:
    words = (vocab + 31) // 32
    dens = lo + uniform_f64(seed, n_states) * (hi - lo)
    table = np.zeros((n_states, words), dtype=np.uint32)
    for s in range(n_states):
        bits = uniform_f64(seed + 1 + s, words * 32) < dens[s]
        bits[0] = True
        bits[vocab:] = False
        table[s] = np.packbits(bits.reshape(words, 32), axis=1, bitorder="little").view(np.uint32).reshape(words)
    return table


def config3(seed=3, rows=128, vocab=151936, n_states=64) -> Workload:
    """Constrained decoding: 64-state table of 1-20 % density (token 0 always allowed); first half
    of the rows greedy, second half T=1 with top-k 20."""
    x = normal_f32(seed, rows * vocab, 2.0).reshape(rows, vocab)
    table = random_mask_table(seed + 500, n_states, vocab)
    state = randint(seed + 600, rows, 0, n_states).astype(np.int32)
    half = rows // 2
    temp = np.concatenate([_const(half, 0.0), _const(rows - half, 1.0)])
    top_k = np.concatenate([_const(half, 0, np.uint32), _const(rows - half, 20, np.uint32)])
    return Workload("config3_grammar", x, temp, top_k, _const(rows, 1.0), _const(rows, 0.0), _const(rows, 0.0),
                    _const(rows, 1.0), None, None, uniform_f32(seed + 3000, rows), mask_words=table,
                    state_flags=np.zeros(n_states, np.uint8), mask_state=state)


def config4(seed=4, rows=256, vocab=256000) -> Workload:
    """Heterogeneous batch: bf16 N(0, 2.5); per-row top-k in [1,1024], top-p in [0.5,1], T in
    [0.3,1.5], repetition in [1,1.3]; 2048-id histories; 30 % of rows under a 5 % bitmask."""
    x = f32_to_bf16_bits(normal_f32(seed, rows * vocab, 2.5)).reshape(rows, vocab)
    u = uniform_f64(seed + 700, rows * 5).reshape(5, rows)
    top_k = (1 + (u[0] * 1024).astype(np.int64)).clip(1, 1024).astype(np.uint32)
    top_p = (0.5 + 0.5 * u[1]).astype(np.float32)
    temp = (0.3 + 1.2 * u[2]).astype(np.float32)
    rep = (1.0 + 0.3 * u[3]).astype(np.float32)
    table = random_mask_table(seed + 500, 4, vocab, 0.05, 0.05)
    state = np.where(u[4] < 0.3, randint(seed + 600, rows, 0, 4), -1).astype(np.int32)
    ho, hi = _history(seed + 1000, rows, 2048, vocab)
    return Workload("config4_hetero_bf16", x, temp, top_k, top_p, _const(rows, 0.0), _const(rows, 0.0), rep, ho, hi,
                    uniform_f32(seed + 3000, rows), mask_words=table, state_flags=np.zeros(4, np.uint8),
                    mask_state=state)


def config5(seed=5, sequences=256, positions=4, vocab=151936) -> Workload:
    """Vocabulary-sharded sampling with 4-token draft verification: sequences x positions f32 rows
    N(0, 2); top-p 0.95 over the per-shard top-64 candidates; seeded draft ids."""
    rows = sequences * positions
    x = normal_f32(seed, rows * vocab, 2.0).reshape(rows, vocab)
    # drafts agree with the true argmax most of the time so that acceptance lengths vary
    am = x.argmax(axis=1).astype(np.uint32)
    flip = uniform_f64(seed + 800, rows) < 0.25
    draft = np.where(flip, randint(seed + 900, rows, 0, vocab).astype(np.uint32), am)
    return Workload("config5_tp_verify", x, _const(rows, 1.0), _const(rows, 0, np.uint32), _const(rows, 0.95),
                    _const(rows, 0.0), _const(rows, 0.0), _const(rows, 1.0), None, None,
                    uniform_f32(seed + 3000, rows), extra={"draft": draft.reshape(sequences, positions),
                                                            "cand": 64})


def headline(seed=7, rows=256, vocab=151936) -> Workload:
    """The shape the headline metric is quoted on: B=256, V=151936 with config 2's per-row recipe."""
    w = config2(seed=seed, rows=rows, vocab=vocab)
    w.name = "headline_b256_v151936_topk50_topp0.9"
    return w
