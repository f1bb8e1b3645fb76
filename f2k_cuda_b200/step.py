"""The attention calls of one denoise step, eagerly or as one CUDA graph.

The reference's transformer runs, per model forward, 8 DoubleStreamBlocks (JointAttention over
separate text and image streams) and then 24 SingleStreamBlocks (Attention over the combined
text||image stream): F2K_CUDA src/backend/cuda/flux_transformer.cu:412-439. With classifier-free
guidance its serving loop runs the model twice per step, on the conditional and then on the
unconditional text embedding (tools/serve.cu:563-566), which doubles the calls. `StepAttention`
issues exactly those calls through the fused entry point (QK-norm + RoPE + attention, two kernels
per call), either one by one or captured once into a CUDA graph and replayed, so that per-step
time can be reported without per-call launch overhead.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .api import Attention, JointAttention


@dataclass
class DoubleCall:
    """Raw projections of one double-stream block: text and image streams, and its outputs."""
    q_txt: torch.Tensor
    k_txt: torch.Tensor
    v_txt: torch.Tensor
    q_img: torch.Tensor
    k_img: torch.Tensor
    v_img: torch.Tensor
    o_txt: torch.Tensor
    o_img: torch.Tensor


@dataclass
class SingleCall:
    """Raw projections of one single-stream block over the combined stream, and its output."""
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    o: torch.Tensor


class StepAttention:
    def __init__(self, batch: int, seq_txt: int, seq_img: int, n_heads: int, head_dim: int = 128):
        self.joint = JointAttention(JointAttention.Config(batch, seq_txt, seq_img, n_heads, head_dim))
        self.single = Attention(Attention.Config(batch, seq_txt + seq_img, n_heads, head_dim))
        self._ok = self.joint.ok() and self.single.ok()
        self.ws_joint = self.ws_single = None
        if self._ok:
            self.ws_joint = torch.empty(self.joint.fused_workspace_size_bytes(), dtype=torch.uint8, device="cuda")
            self.ws_single = torch.empty(self.single.fused_workspace_size_bytes(), dtype=torch.uint8, device="cuda")
        self._graph = None

    def ok(self) -> bool:
        return self._ok

    def last_error(self) -> str:
        return self.joint.last_error() or self.single.last_error()

    def device_status(self) -> int:
        return self.joint.device_status() | self.single.device_status()

    def run(self, passes, gammas, tables, tables_combined, eps: float = 1e-6, stream=None) -> int:
        """passes: one (double_calls, single_calls) pair per model forward of the step - one pair
        without guidance, two (conditional, unconditional) with it. gammas = (gq_txt, gk_txt,
        gq_img, gk_img); tables = (cos_txt, sin_txt, cos_img, sin_img) for the double blocks,
        tables_combined = (cos, sin) over text||image for the single blocks, which use the image
        stream's gains (the reference's single blocks have one gain pair). Returns the number of
        attention calls issued; raises on a refused call."""
        n = 0
        for doubles, singles in passes:
            for c in doubles:
                if not self.joint.forward_fused(c.q_txt, c.k_txt, c.v_txt, c.q_img, c.k_img, c.v_img, gammas, tables, eps,
                                                c.o_txt, c.o_img, self.ws_joint, stream):
                    raise RuntimeError(self.joint.last_error())
                n += 1
            for c in singles:
                if not self.single.forward_fused(None, None, None, c.q, c.k, c.v, (None, None, gammas[2], gammas[3]),
                                                 (None, None, *tables_combined), eps, None, c.o, self.ws_single, stream):
                    raise RuntimeError(self.single.last_error())
                n += 1
        return n

    def capture(self, passes, gammas, tables, tables_combined, eps: float = 1e-6):
        """Runs the step once eagerly (tensor maps are built, kernels loaded), then records it into a
        CUDA graph on a side stream. Returns (graph, calls); graph.replay() re-issues the step."""
        calls = self.run(passes, gammas, tables, tables_combined, eps)
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                self.run(passes, gammas, tables, tables_combined, eps, stream=side)
        torch.cuda.synchronize()
        self._graph = graph
        return graph, calls
