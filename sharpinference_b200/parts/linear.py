"""Matrix products of the parts: ``y = a . W^T`` with the weight stored ``[out, in]``.

Which routine runs is decided by the weight's dtype, not by a global mode:

* float32 weight: the CUDA-core kernel with float32 accumulation (``gemm_generic.cu``), the
  product of the true 32-bit path; no tensor cores and no reduced-precision mode are involved.
* bfloat16 weight: a tensor-core product with float32 accumulation and float32 output.  With
  many rows (prompt portions) the dense ones go to the vendor library through ``torch.mm``, which
  is where the reference uses a library too (cublasGemmEx for batched projections,
  src/SharpInference.Cuda/CudaBackend.cs:2083-2117); with few rows (decode), where the reference
  runs its own matvec kernels (llm_matvec_*, src/SharpInference.Cuda/CudaTextKernels.cs:1325), they
  can run our tcgen05 weight-streaming kernel (``stream_rows``; the library stays the default there
  because it measured faster); sizes neither takes (an inner size that is no multiple of 8) use the
  CUDA-core kernel.

The grouped (per-expert) product has no library counterpart and always runs our own kernels.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops


class Linear:
    """A weight ``[out, in]``, an optional bias ``[out]`` (float32) and the product with them.  Output is
    float32 ``[M, out]``.  The reference adds a projection's bias where a model stores one
    (src/SharpInference.Core/ModelGraph.cs:269-270 probes for it)."""

    def __init__(self, weight: torch.Tensor, name: str = "", stream_rows: int = 0,
                 bias: Optional[torch.Tensor] = None):
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
        # Up to this many rows the product runs on our weight-streaming tcgen05 kernel instead of the
        # library.  Off by default: measured on B200 at Scout sizes the library's split-K kernels are about
        # 20 % faster on these shapes (qkv 14 vs 18 us, shared gate|up 28 vs 37 us at 8 rows).
        self.stream_rows = stream_rows

    def __call__(self, a: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
        """``a . W^T`` into ``out``, or added to it (``accumulate``).  Only the product that :meth:`streams`
        adds with reductions, so that another kernel may add into the same ``out`` at the same time."""
        if accumulate:
            if out is None:
                raise ValueError("accumulate needs an output to add to")
            if self.streams(a):
                return ops.tc_dense(a, self.weight, out=out, accumulate=True)
            return out.add_(self(a))
        w = self.weight
        if w.dtype == torch.float32:
            if a.dtype != torch.float32:
                a = a.to(torch.float32)
            return ops.gemm_nt(a, w, out=out, bias=self.bias)
        if self._use_library and a.dtype == torch.bfloat16:
            if self.streams(a):
                y = ops.tc_dense(a, w, out=out)
            elif out is not None:
                y = torch.mm(a, self._wt, out_dtype=torch.float32, out=out)
            else:
                y = torch.mm(a, self._wt, out_dtype=torch.float32)
            return ops.add_bias(y, self.bias) if self.bias is not None else y
        return ops.gemm_nt(a, w, out=out, bias=self.bias)

    def streams(self, a: torch.Tensor) -> bool:
        """Whether this product of ``a`` would run on the weight-streaming tensor-core kernel."""
        return (self._use_library and self.bias is None and a.dtype == torch.bfloat16
                and a.shape[0] <= self.stream_rows)


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
