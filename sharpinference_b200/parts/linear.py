"""Matrix products of the parts: ``y = a . W^T`` with the weight stored ``[out, in]``.

Which routine runs is decided by the weight's dtype and the number of rows, not by a global mode:

* float32 weight: the CUDA-core kernel with float32 accumulation (``gemm_generic.cu``), the
  product of the true 32-bit path; no tensor cores and no reduced-precision mode are involved.
* bfloat16 weight: a tensor-core product with float32 accumulation and float32 output.  The dense ones go to
  the vendor library through ``torch.mm``, which is where the reference uses a library too (cublasGemmEx for
  batched projections, src/SharpInference.Cuda/CudaBackend.cs:2083-2117).  With few rows (decode), where the
  reference runs matvec kernels of its own (llm_matvec_*, src/SharpInference.Cuda/CudaTextKernels.cs:1325),
  they can run the engine's weight-streaming kernel instead (``stream_rows``; ``dense_rows.cu``: the weight is
  read once, rows dealt evenly over the SMs, bias, add-in or SwiGLU in its epilogue).  Alone that kernel is the
  faster one on B200 (see DEFAULT_STREAM_ROWS); inside a decode step it is not, so the library is the default.
* sizes neither takes (an inner size that is no multiple of 8) use the CUDA-core kernel.

The grouped (per-expert) product has no library counterpart and always runs our own kernels.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops


# Rows up to which a bfloat16 product runs on the weight-streaming kernel by default: none.  Measured on B200
# at Scout sizes, microseconds at 1 to 8 rows, own kernel / library, alone and between two other kernels of a
# captured graph: qkv 7168 x 5120 12.8 / 14.4, o 5120 x 5120 9.9 / 11.8, shared down 5120 x 8192 14.8 / 17.5,
# shared gate|up with SwiGLU 27.0 / 29.9 (library product plus the SwiGLU kernel).  In a decode step of 8 layers
# the own kernel on every product gives 593 against 614 tokens a second at batch 1 and 2198 against 2221 at
# batch 8: it deals its rows over exactly as many CTAs as fit the SMs at once, with all their registers, so a
# kernel of another stream (the router beside the shared expert) or a block of a neighbour that is still or
# already there delays one of its CTAs by up to the whole product.
DEFAULT_STREAM_ROWS = 0


class Linear:
    """A weight ``[out, in]``, an optional bias ``[out]`` (float32) and the product with them.  Output is
    float32 ``[M, out]``.  The reference adds a projection's bias where a model stores one
    (src/SharpInference.Core/ModelGraph.cs:269-270 probes for it)."""

    def __init__(self, weight: torch.Tensor, name: str = "", stream_rows: int = DEFAULT_STREAM_ROWS,
                 bias: Optional[torch.Tensor] = None, split_add_rows: int = 0):
        if weight.dim() != 2:
            raise ValueError(f"linear weight '{name}' must be 2-D, found shape {tuple(weight.shape)}")
        if bias is not None and tuple(bias.shape) != (weight.shape[0],):
            raise ValueError(f"bias of '{name}' has shape {tuple(bias.shape)}, expected ({weight.shape[0]},)")
        self.weight = weight
        self.bias = bias
        self.name = name
        self.out_features, self.in_features = weight.shape
        self._use_library = (weight.dtype == torch.bfloat16 and self.in_features % 8 == 0)
        self._wt = weight.t() if self._use_library else None
        # Up to this many rows (at most ops.DENSE_ROWS_MAX) the product runs on the weight-streaming kernel
        # instead of the library; 0: the library at every size.
        self.stream_rows = stream_rows
        # Up to this many rows an add-in (``accumulate``) runs on the grouped tensor-core kernel with one group
        # and K cut over CTAs: small CTAs that add with reductions and run well beside other kernels.
        self.split_add_rows = split_add_rows

    def __call__(self, a: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
        """``a . W^T`` into ``out``, or added to it (``accumulate``).  Where :meth:`adds_with_reductions` says so
        the add-in is done with reductions, so that another kernel may add into the same ``out`` at the same
        time; otherwise it is the product followed by an addition."""
        if accumulate:
            if out is None:
                raise ValueError("accumulate needs an output to add to")
            if self.adds_with_reductions(a):
                if a.shape[0] <= self.split_add_rows:
                    return ops.tc_dense(a, self.weight, out=out, accumulate=True)
                return ops.dense_rows(a, self.weight, out=out, accumulate=True)
            return out.add_(self(a))
        w = self.weight
        if w.dtype == torch.float32:
            if a.dtype != torch.float32:
                a = a.to(torch.float32)
            return ops.gemm_nt(a, w, out=out, bias=self.bias)
        if self._use_library and a.dtype == torch.bfloat16:
            if self.streams(a):
                return ops.dense_rows(a, w, out=out, bias=self.bias)
            if out is not None:
                y = torch.mm(a, self._wt, out_dtype=torch.float32, out=out)
            else:
                y = torch.mm(a, self._wt, out_dtype=torch.float32)
            return ops.add_bias(y, self.bias) if self.bias is not None else y
        return ops.gemm_nt(a, w, out=out, bias=self.bias)

    def streams(self, a: torch.Tensor) -> bool:
        """Whether this product of ``a`` runs on the weight-streaming kernel."""
        return (self._use_library and a.dtype == torch.bfloat16
                and a.shape[0] <= min(self.stream_rows, ops.DENSE_ROWS_MAX))

    def adds_with_reductions(self, a: torch.Tensor) -> bool:
        """Whether ``accumulate`` adds this product of ``a`` into the output element by element with reductions
        (one of the engine's own kernels) rather than as a product followed by an addition."""
        return (self._use_library and self.bias is None and a.dtype == torch.bfloat16
                and (a.shape[0] <= self.split_add_rows or self.streams(a)))


class GroupedLinear:
    """Per-expert weights ``[E, out, in]``; rows arrive sorted by expert."""

    def __init__(self, weight: torch.Tensor, name: str = ""):
        if weight.dim() != 3:
            raise ValueError(f"grouped weight '{name}' must be [E, out, in], found shape {tuple(weight.shape)}")
        self.weight = weight
        self.name = name
        self.num_groups, self.out_features, self.in_features = weight.shape

    def __call__(self, a: torch.Tensor, group_offsets: torch.Tensor, *, rows: int,
                 a_rows: Optional[torch.Tensor] = None, out_rows: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
        if self.weight.dtype == torch.float32 and a.dtype != torch.float32:
            a = a.to(torch.float32)
        return ops.gemm_nt(a, self.weight, out=out, group_offsets=group_offsets, a_rows=a_rows, out_rows=out_rows,
                           rows=rows, accumulate=accumulate)
