"""The runtime a model runs on: device, compute type, and the choice of kernel per operation.

Two modes.  ``float32``: every tensor and every sum is 32-bit, matrix products by
the fixed-order FMA kernel, attention by the general kernel; nothing uses tensor cores
or a reduced-precision matrix mode.  ``bfloat16``: weights, activations between
kernels and the cache are bfloat16; the residual stream, norms, softmax, rotation
angles and logits stay float32.
"""
from __future__ import annotations

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
