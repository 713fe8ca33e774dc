"""Stack-level runner: a whole stack of quantized linears replayed as ONE CUDA graph.

Decode-time (M <= 16) layers take 3-25 us each on a B200, so launch gaps and per-call
allocations dominate a Python loop over ``BlkQ4Linear.forward`` (the reference module
allocates its output per call and launches on the legacy default stream,
python/ms_blkq4linear_ext/ms_blkq4linear.cpp:58,107).  ``LinearStack`` owns a
persistent workspace (one buffer per named activation), wires each layer to an input and
an output buffer, captures the whole pass once per row count M on its own stream, and
replays it.  Inside the graph the skinny kernels are launched with
``BLKQ4_GEMM_EARLY_WEIGHT_FETCH``: the weights of layer i+1 stream in while layer i
drains.

It runs the linears only: what sits between them in a model (attention, activation
functions, norms) is the caller's and can be captured into the same graph by passing
``between`` hooks.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .ms_blkq4linear import BlkQ4Linear


class LinearStack:
    """``steps`` = [(layer, input buffer name, output buffer name), ...] executed in order.

    Buffer ``"x"`` is the stack's input ([M, in_features of the first reader]); every other
    name is created on first use as an output and can be read by later steps.
    """

    def __init__(self, steps: Sequence[Tuple[BlkQ4Linear, str, str]],
                 between: Optional[Dict[int, Callable[[Dict[str, torch.Tensor]], None]]] = None):
        self.steps = list(steps)
        self.between = dict(between or {})
        self._graphs: Dict[int, Tuple[torch.cuda.CUDAGraph, Dict[str, torch.Tensor]]] = {}
        self.device = self.steps[0][0].q_weights.device
        self.stream = torch.cuda.Stream(self.device)
        written = {"x"}
        for lyr, src, dst in self.steps:
            if src not in written:
                raise ValueError(f"step reads buffer {src!r} before anything wrote it")
            written.add(dst)

    # ---- workspace ----
    def _workspace(self, M: int) -> Dict[str, torch.Tensor]:
        bufs: Dict[str, torch.Tensor] = {}
        for lyr, src, dst in self.steps:
            if src not in bufs:
                bufs[src] = torch.zeros(M, lyr.in_features, dtype=torch.float16, device=self.device)
            elif bufs[src].size(1) != lyr.in_features:
                raise ValueError(f"buffer {src!r} has width {bufs[src].size(1)}, layer wants {lyr.in_features}")
            if dst not in bufs:
                bufs[dst] = torch.zeros(M, lyr.out_features, dtype=torch.float16, device=self.device)
            elif bufs[dst].size(1) != lyr.out_features:
                raise ValueError(f"buffer {dst!r} has width {bufs[dst].size(1)}, layer writes {lyr.out_features}")
        return bufs

    def _run_eager(self, bufs):
        for i, (lyr, src, dst) in enumerate(self.steps):
            lyr(bufs[src], out=bufs[dst])
            hook = self.between.get(i)
            if hook is not None:
                hook(bufs)

    def _capture(self, M: int):
        bufs = self._workspace(M)
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream):
            for _ in range(2):  # the first pass settles every layer (plain launches), the second warms up
                self._run_eager(bufs)
        self.stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=self.stream):
            self._run_eager(bufs)
        self._graphs[M] = (graph, bufs)
        return self._graphs[M]

    # ---- public ----
    def buffers(self, M: int) -> Dict[str, torch.Tensor]:
        """The persistent workspace for row count M (captures the graph on first use)."""
        return (self._graphs.get(M) or self._capture(M))[1]

    def replay(self, M: int):
        """One pass over the stack on the current stream; reads ``buffers(M)["x"]``."""
        graph, _ = self._graphs.get(M) or self._capture(M)
        graph.replay()

    def forward(self, x: torch.Tensor, result: str) -> torch.Tensor:
        """Copy ``x`` into the input buffer, replay, return the buffer named ``result``."""
        M = x.size(0)
        _, bufs = self._graphs.get(M) or self._capture(M)
        bufs["x"].copy_(x)
        self.replay(M)
        return bufs[result]

    @property
    def num_linears(self) -> int:
        return len(self.steps)

    def weight_bytes(self) -> int:
        return sum(l.q_weights.numel() + 2 * l.q_scales.numel() + l.q_zp.numel() for l, _, _ in self.steps)


def llama_like_stack(hidden: int, ffn: int, blocks: int, block_size: int, col_wise: bool, scale_only: bool,
                     device, sigma: float = 0.02, seed: int = 0, weight_fn=None) -> LinearStack:
    """The seven linears of a Llama-style decoder block, ``blocks`` times, with random weights:
    q, k, v, o (hidden -> hidden), gate, up (hidden -> ffn), down (ffn -> hidden).  Shapes only:
    q/k/v/gate/up read the block input, o reads q's output and down reads gate's output, so every
    buffer a layer reads was produced inside the graph (true stream-order dependencies), and the
    block's output ("h") is o's and down's sum stand-in: down writes it."""
    steps: List[Tuple[BlkQ4Linear, str, str]] = []
    g = torch.Generator().manual_seed(seed)

    def make(n, k):
        w = weight_fn(n, k) if weight_fn else (torch.randn(n, k, generator=g) * sigma).to(torch.float16)
        return BlkQ4Linear(block_size, col_wise, scale_only, w.to(device))

    src = "x"
    for b in range(blocks):
        steps += [(make(hidden, hidden), src, "q"), (make(hidden, hidden), src, "k"), (make(hidden, hidden), src, "v"),
                  (make(hidden, hidden), "q", "o"), (make(ffn, hidden), "o", "gate"), (make(ffn, hidden), "o", "up"),
                  (make(hidden, ffn), "gate", f"h{b % 2}")]
        src = f"h{b % 2}"
    return LinearStack(steps)
