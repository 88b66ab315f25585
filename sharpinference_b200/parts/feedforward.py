"""Feed-forward parts: dense SwiGLU, and a top-1 sigmoid-routed mixture of experts with an
always-on shared expert.

Dense (src/SharpInference.Engine/ForwardPass.cs:2006-2015): ``y = (silu(h Wg^T) * (h Wu^T)) Wd^T``.

Mixture (src/SharpInference.Engine/ForwardPass.cs:2021-2098): router logits ``r = h Wr^T``,
``p = sigmoid(r)``, the expert with the largest ``p`` (first wins), ``w = p[e]``; the routed
expert computes ``(silu(w g) * (w u)) Wd[e]^T`` with ``g = h Wg[e]^T``, ``u = h Wu[e]^T`` (the
weight scales gate and up, which is scaling the expert's input); the shared expert is a dense
SwiGLU on the unscaled ``h``; the two are summed.  Routing stays on the device: the step's rows
are sorted by expert and each expert multiplies its rows in one grouped product.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import FeedForward, StepContext, register_part
from .linear import GroupedLinear, Linear


@register_part("feed_forward", "dense_swiglu")
class DenseSwiGLU(FeedForward):
    graph_safe = True        # reads the step through device tensors only: may be captured in a CUDA graph
    def __init__(self, *, gate_up: Linear, down: Linear, act_dtype: torch.dtype = torch.bfloat16):
        if gate_up.out_features != 2 * down.in_features:
            raise ValueError(f"fused gate|up weight has {gate_up.out_features} rows, expected 2 * {down.in_features}")
        self.gate_up, self.down, self.act_dtype = gate_up, down, act_dtype

    def forward(self, ctx: StepContext, h: torch.Tensor, h32: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
        if self.act_dtype == torch.bfloat16 and self.gate_up.streams(h) and self.gate_up.bias is None:
            act = ops.dense_rows(h, self.gate_up.weight, swiglu=True)     # SwiGLU in the product's epilogue
        else:
            act = ops.swiglu(self.gate_up(h), self.act_dtype)
        return self.down(act, out=out, accumulate=accumulate)


_side_streams: dict = {}


def _side_stream(device: torch.device) -> "torch.cuda.Stream":
    """The second stream of a device, on which the shared expert runs beside the routed ones."""
    key = torch.device(device).index
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=device)
    return _side_streams[key]


def _urgent_stream(device: torch.device) -> "torch.cuda.Stream":
    """A stream of higher priority for short kernels that a longer chain waits for."""
    key = ("urgent", torch.device(device).index)
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=device, priority=-1)
    return _side_streams[key]


@register_part("feed_forward", "moe_sigmoid_top1")
class MoESigmoidTop1(FeedForward):
    wants_fp32_input = True
    graph_safe = True
    # Steps of more rows than this keep the routed gate|up product on the routing's stream (see forward).
    SMALL_STEP_ROWS = 256
    # Up to this many rows the shared expert's down product adds into the output on the grouped tensor-core
    # kernel (one group, K cut over CTAs) instead of the library's product and an addition: alone the library is
    # a little faster on that shape, but beside the routed gate|up product the step is not (Scout sizes, 8
    # layers: batch 1 614 -> 644 tok/s; no difference from batch 8 on).  Both experts then add into a zeroed
    # output with reductions and no longer wait for each other.
    SHARED_DOWN_SPLIT_ADD_ROWS = 4

    def __init__(self, *, router: torch.Tensor, experts_gate_up: GroupedLinear, experts_down: GroupedLinear,
                 shared: Optional[DenseSwiGLU], act_dtype: torch.dtype = torch.bfloat16):
        E = experts_gate_up.num_groups
        if router.shape != (E, experts_gate_up.in_features):
            raise ValueError(f"router weight is {tuple(router.shape)}, expected [{E}, {experts_gate_up.in_features}]")
        if experts_down.num_groups != E or experts_gate_up.out_features != 2 * experts_down.in_features:
            raise ValueError("expert gate|up and down weights disagree on the number or width of the experts")
        self.router = router
        self.experts_gate_up, self.experts_down = experts_gate_up, experts_down
        self.shared = shared
        shared_down = getattr(shared, "down", None)
        if isinstance(shared_down, Linear) and shared_down.split_add_rows == 0:
            shared_down.split_add_rows = self.SHARED_DOWN_SPLIT_ADD_ROWS
        self.num_experts = E
        self.act_dtype = act_dtype
        # the tensor-core path takes bfloat16 weights whose inner sizes are multiples of 8 (TMA rows
        # must start on 16 bytes); everything else runs the CUDA-core kernels
        self._tensor_core = (experts_gate_up.weight.dtype == torch.bfloat16
                             and experts_down.weight.dtype == torch.bfloat16 and act_dtype == torch.bfloat16
                             and experts_gate_up.in_features % 8 == 0 and experts_down.in_features % 8 == 0)

    def forward(self, ctx: StepContext, h: torch.Tensor, h32: Optional[torch.Tensor] = None) -> torch.Tensor:
        T = h.shape[0]
        if h32 is None:
            h32 = h.to(torch.float32)
        # The shared expert and the routed ones meet only where the routed outputs are added, so the shared
        # expert runs on a second stream (inside a graph capture: a fork and a join), forked off before the
        # routing, and the streams join before the routed down product.  Routing, sorting and gathering are
        # short kernels that everything routed waits for, and behind the shared product's many blocks they
        # would queue, so they run on a third stream of higher priority.  Small steps: the routed gate|up
        # product returns to the main stream and streams its weights beside the shared expert's (two streams
        # of weights keep the memory system busier than one; with priority over the shared expert it measured
        # slower).  Large steps: every product fills the GPU by itself; the routed gate|up product stays on the
        # third stream and takes over the SMs as the shared expert's products drain.
        # When the shared expert's down product adds with reductions too (few rows, see SHARED_DOWN_SPLIT_ADD_ROWS),
        # both experts add into a zeroed output and the streams need not meet before the end: each element is
        # 0 + a + b in one order or the other, which is the same number.
        tensor_core = self._tensor_core and h.dtype == torch.bfloat16
        main = torch.cuda.current_stream(h.device)
        side = routed = None
        apart = False
        if self.shared is not None:
            shared_down = getattr(self.shared, "down", None)
            apart = tensor_core and isinstance(shared_down, Linear) and shared_down.adds_with_reductions(h)
            make = torch.zeros if apart else torch.empty
            y = make((T, self.experts_down.out_features), dtype=torch.float32, device=h.device)
            side, routed = _side_stream(h.device), _urgent_stream(h.device)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                if apart:
                    self.shared.forward(ctx, h, out=y, accumulate=True)
                else:
                    self.shared.forward(ctx, h, out=y)
            routed.wait_stream(main)
        else:
            y = torch.zeros((T, self.experts_down.out_features), dtype=torch.float32, device=h.device)
        act = None
        with torch.cuda.stream(routed if routed is not None else main):
            expert, weight, _, offsets, sorted_rows = ops.router_top1(h32, self.router, sort=True)
            # one row is its own sorted order: nothing to gather
            h_sorted = (h if T == 1 else ops.gather_rows_bf16(h, sorted_rows)) if tensor_core else None
            if tensor_core and T > self.SMALL_STEP_ROWS:
                act = ops.tc_grouped_gemm(h_sorted, self.experts_gate_up.weight, offsets, mode=ops.TC_MODE_SWIGLU,
                                          row_scale=weight, scale_rows=sorted_rows)
        if routed is not None:
            main.wait_stream(routed)
        if "router_choices" in ctx.extras:          # tracing: which expert every row went to
            ctx.extras["router_choices"].append(expert)
        if tensor_core:
            if act is None:
                act = ops.tc_grouped_gemm(h_sorted, self.experts_gate_up.weight, offsets, mode=ops.TC_MODE_SWIGLU,
                                          row_scale=weight, scale_rows=sorted_rows)
            if side is not None and not apart:
                main.wait_stream(side)
            ops.tc_grouped_gemm(act, self.experts_down.weight, offsets, mode=ops.TC_MODE_STORE, out=y,
                                out_rows=sorted_rows, accumulate=True)
            if apart:
                main.wait_stream(side)
            return y
        gu = self.experts_gate_up(h, offsets, rows=T, a_rows=sorted_rows)          # sorted order
        act = ops.swiglu(gu, self.act_dtype, row_scale=weight, scale_rows=sorted_rows)
        if side is not None:
            main.wait_stream(side)
        self.experts_down(act, offsets, rows=T, out_rows=sorted_rows, out=y, accumulate=True)
        return y
