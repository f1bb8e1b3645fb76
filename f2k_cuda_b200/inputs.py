"""Seeded synthetic inputs of the joint-attention workloads (shapes of the FLUX.2-klein MMDiT).

Values come from a counter-based generator (splitmix64 of seed, stream id and element index,
then Box-Muller), so every tensor is reproducible bit for bit on any machine and does not
depend on a library's random stream. Distributions: Q, K, V ~ N(0, 1) rounded to bf16; QK-norm
gains 1 + U(-0.1, 0.1); RoPE theta 2000 over axes (t, h, w, l) of 32 dims each; text tokens at
(0, 0, 0, l), image tokens at (t, h, w, 0) row-major over a square grid, one t per image.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

AXES_DIM = (32, 32, 32, 32)
ROPE_THETA = 2000.0
RMS_EPS = 1e-6
SEED_BASE = 0xF2C0DE00


@dataclass(frozen=True)
class Workload:
    name: str
    batch: int
    seq_txt: int
    img_grids: tuple          # one (rows, cols) grid per image; the i-th image sits at t = i
    n_heads: int = 32
    head_dim: int = 128
    seed: int = SEED_BASE

    @property
    def seq_img(self) -> int:
        return sum(r * c for r, c in self.img_grids)

    @property
    def seq(self) -> int:
        return self.seq_txt + self.seq_img

    @property
    def flops(self) -> float:
        """4 * B * H * S^2 * D: QK^T and PV, two flops per multiply-add."""
        return 4.0 * self.batch * self.n_heads * self.seq ** 2 * self.head_dim


# The five configurations the headline metric is quoted on, in order.
WORKLOADS = {
    "s1152": Workload("s1152", 1, 128, ((32, 32),), seed=SEED_BASE + 0),
    "s4608": Workload("s4608", 1, 512, ((64, 64),), seed=SEED_BASE + 1),
    "s4608_b4": Workload("s4608_b4", 4, 512, ((64, 64),), seed=SEED_BASE + 2),
    "s8704_edit": Workload("s8704_edit", 1, 512, ((64, 64), (64, 64)), seed=SEED_BASE + 3),
    "s16896": Workload("s16896", 1, 512, ((128, 128),), seed=SEED_BASE + 4),
}

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = x + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def uniform01(seed: int, stream: int, n: int) -> np.ndarray:
    """n doubles in (0, 1), a pure function of (seed, stream, index)."""
    with np.errstate(over="ignore"):
        key = _splitmix64(np.array([seed & 0xFFFFFFFFFFFFFFFF], np.uint64) ^
                          (np.uint64(stream) * np.uint64(0xD1342543DE82EF95)))
        bits = _splitmix64(key + np.arange(n, dtype=np.uint64))
    return ((bits >> np.uint64(11)).astype(np.float64) + 0.5) * (1.0 / 9007199254740992.0)


def normal(seed: int, stream: int, n: int) -> np.ndarray:
    """n standard normals (float32) by Box-Muller on two uniform streams."""
    u1 = uniform01(seed, 2 * stream, n)
    u2 = uniform01(seed, 2 * stream + 1, n)
    return (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)).astype(np.float32)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    return ((u + r) >> np.uint32(16)).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def token_positions(w: Workload):
    """(txt_positions [seq_txt, 4], img_positions [seq_img, 4]) as the reference lays them out
    (F2K_CUDA src/backend/cuda/flux_transformer.cu:288-319); image i of an edit shape has t = i."""
    txt = np.zeros((w.seq_txt, 4), np.int32)
    txt[:, 3] = np.arange(w.seq_txt)
    parts = []
    for t, (rows, cols) in enumerate(w.img_grids):
        s = np.arange(rows * cols)
        p = np.zeros((rows * cols, 4), np.int32)
        p[:, 0], p[:, 1], p[:, 2] = t, s // cols, s % cols
        parts.append(p)
    return txt, np.concatenate(parts, 0)


@dataclass
class Problem:
    """Host-side tensors of one workload: bf16 bit patterns (uint16) and fp32 tables."""
    w: Workload
    q_txt: np.ndarray; k_txt: np.ndarray; v_txt: np.ndarray
    q_img: np.ndarray; k_img: np.ndarray; v_img: np.ndarray
    gammas: tuple = field(default=())   # gq_txt, gk_txt, gq_img, gk_img
    pos_txt: np.ndarray = None
    pos_img: np.ndarray = None


def make_problem(w: Workload, dist: str = "normal", heads: int | None = None) -> Problem:
    """Draw order: q_txt, k_txt, v_txt, q_img, k_img, v_img, then the four gains.
    dist "uniform" gives U(-0.5, 0.5), the distribution of the reference's own tests.
    `heads` restricts the head count (values of head h do not depend on it)."""
    H = w.n_heads if heads is None else heads
    D = w.head_dim

    def draw(stream, seq):
        n = w.batch * seq * w.n_heads * D
        x = normal(w.seed, stream, n) if dist == "normal" else \
            (uniform01(w.seed, 100 + stream, n) - 0.5).astype(np.float32)
        x = x.reshape(w.batch, seq, w.n_heads, D)[:, :, :H]
        return to_bf16_bits(np.ascontiguousarray(x))

    t = [draw(i, w.seq_txt) for i in range(3)]
    im = [draw(3 + i, w.seq_img) for i in range(3)]
    gam = tuple(to_bf16_bits((1.0 + 0.2 * (uniform01(w.seed, 50 + i, D) - 0.5)).astype(np.float32))
                for i in range(4))
    pt, pi = token_positions(w)
    return Problem(w, *t, *im, gammas=gam, pos_txt=pt, pos_img=pi)
