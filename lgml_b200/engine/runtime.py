"""The runtime a model runs on: device, compute type, and the choice of kernel per operation.

Two modes.  ``float32``: every tensor and every sum is 32-bit, matrix products by
the fixed-order FMA kernel, attention by the general kernel; nothing uses tensor cores
or a reduced-precision matrix mode.  ``bfloat16``: weights, activations between
kernels and the cache are bfloat16; the residual stream, norms, softmax, rotation
angles and logits stay float32.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .. import ops

_STATUS_TEXT = {
    1: "a token id was outside the vocabulary",
    2: "a key/value write had no page in the block table",
    3: "attention met a position without a page in the block table",
    10: "a tensor-core matrix product gave up waiting for its own copies or products",
    12: "the tensor-core prompt attention (one tile per CTA) gave up waiting for its own copies or products",
    13: "the tensor-core prompt attention (two tiles per CTA) gave up waiting for its own copies or products",
}


AHEAD_BYTES = 24 << 20      # weights asked of L2 ahead, per layer (measured best at 24 to 32 MiB)
AHEAD_MAX_BATCH = 4         # ... in captured steps of at most this many requests (at 8 the step gets slower)
MAX_RESULT = 4096     # most sampled rows of a step whose ids travel with the status word


class DeviceFault(RuntimeError):
    """A kernel flagged an input it refused to use (it skipped the access)."""


class Runtime:
    def __init__(self, device="cuda:0", dtype: torch.dtype = torch.bfloat16, gemm: str = "auto"):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError(f"the engine runs on a CUDA device only, not on '{device}'")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is available; the engine has no CPU path")
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"compute type must be bfloat16 or float32, not {dtype}")
        self.dtype = dtype
        torch.cuda.set_device(self.device)
        # sampled token ids of a step end at result[MAX_RESULT], where the status word sits: one
        # copy brings both to the host
        self.result = torch.zeros(MAX_RESULT + 1, dtype=torch.int32, device=self.device)
        self.status = self.result[MAX_RESULT:]
        self.gemm_backend = gemm
        self.attention_backend = "auto"
        # Asking L2 for weights ahead of their reader: only inside a captured decode step of few
        # requests, which sets ``side`` (a stream beside the step's chain) for the capture.
        self.ahead_bytes = 0 if os.environ.get("LGML_L2_AHEAD") == "0" else AHEAD_BYTES
        self.side: Optional[torch.cuda.Stream] = None
        self._forked = False

    # ---- matrix products ---------------------------------------------------------------
    def linear(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
               out_dtype: Optional[torch.dtype] = None, partials_ok: bool = False):
        """y = x . w^T (+ bias); x [M,K], w [N,K] in the compute type, y in ``out_dtype``.
        With ``partials_ok`` the caller accepts ``ops.Partials`` (the partial sums of a product
        cut along K, which the next kernel adds up) in place of a tensor."""
        out_dtype = out_dtype or self.dtype
        if self.dtype == torch.float32:
            out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=x.device)
            return ops.gemm_f32(x, w, out, bias)
        return ops.gemm_bf16(x, w, out_dtype, bias, backend=self.gemm_backend, status=self.status, partials_ok=partials_ok)

    def ahead(self, tensors) -> None:
        """Ask L2 for the first ``ahead_bytes`` of ``tensors`` (weights that the step reads a few
        kernels from now), on the side stream, from this point of the step's chain on.  While a
        layer's attention runs HBM is mostly idle at small batches, and a product that finds the
        head of its weights in L2 ends that much earlier.  Outside a capture that set ``side``
        this does nothing."""
        if self.side is None or not self.ahead_bytes:
            return
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        self.side.wait_event(ev)
        left = self.ahead_bytes
        with torch.cuda.stream(self.side):
            for t in tensors:
                n = min(left, t.numel() * t.element_size())
                if n >= 16:
                    ops.l2_ahead(t, n, keep=True)
                left -= n
        self._forked = True

    def join(self) -> None:
        """The step's stream waits for what ``ahead`` put on the side stream (a capture must end so)."""
        if self._forked:
            torch.cuda.current_stream().wait_stream(self.side)
            self._forked = False

    def fused_swiglu(self, x: torch.Tensor, w_pairs: torch.Tensor) -> bool:
        """Whether the gated feed-forward can run its first product and activation as one kernel."""
        return self.dtype == torch.bfloat16 and self.gemm_backend in ("auto", "tcgen05") and ops.tcgen05_supports(x, w_pairs)

    # ---- attention ---------------------------------------------------------------------
    def attention(self, q, batch, cache, out, n_heads: int, scale: float, window: int, softcap: float = 0.0) -> torch.Tensor:
        """Attention of the step's queries over the cache.  A cap on the scores (``softcap`` > 0)
        is known to the general kernel only, so it takes that kernel in both compute types."""
        if self.dtype == torch.float32 or self.attention_backend == "ref" or softcap:
            return ops.paged_attention_ref(q, batch.positions, batch.seq_of_token, cache.block_table, cache.k, cache.v,
                                           out, n_heads, scale, window, self.status, softcap=softcap)
        return ops.paged_attention(q, batch, cache, out, n_heads, scale, window, self.status)

    # ---- faults ------------------------------------------------------------------------
    def check_status(self, code: Optional[int] = None) -> None:
        """Raise if a kernel flagged a fault; ``code`` is the status word when the caller
        already has it on the host."""
        if code is None:
            code = int(self.status.item())
        if code:
            self.status.zero_()
            raise DeviceFault(f"kernel status {code}: {_STATUS_TEXT.get(code, 'unknown')}")
