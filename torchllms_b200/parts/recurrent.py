"""Recurrent mixers: a state of fixed size per request instead of a cache that grows.

The state lives in the cache manager's state rows (one row per live request, zeroed when the
request is admitted), in 32-bit floats whatever the activation dtype; a prompt portion runs the
recurrence over its tokens inside one kernel and leaves the state for the next step.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels.lazy import PendingProduct
from ..weights.loader import ExpectedTensor
from .base import BuildEnv, Mixer, StateNeed, as_compute, register_mixer


@register_mixer("mingru")
class MinGRU(Mixer):
    """A gated recurrence whose gates read only the current token:

        ``z_t = sigmoid(Wz x_t + bz)``,  ``u_t = Wx x_t + bx``,
        ``c_t = u_t + 1/2`` where ``u_t >= 0``, ``sigmoid(u_t)`` elsewhere,
        ``S_t = (1 - z_t) S_(t-1) + z_t c_t``   (element by element, ``S`` of size ``width``),
        output ``Wo (S_t * silu(Wg x_t))``.

    The three projections of the input are one stacked product; the gates, the candidate, the
    recurrence and the output gate are one kernel in float32; ``Wo`` is left to whoever adds the
    result to the stream."""

    graph_safe = True

    def __init__(self, env: BuildEnv, *, dim: int, width: int):
        self.env = env
        self.dim, self.width = int(dim), int(width)
        if self.width <= 0:
            raise ValueError(f"the width of a recurrent state must be positive, got {width}")
        self.w_in: Optional[torch.Tensor] = None
        self.b_in: Optional[torch.Tensor] = None
        self.wo: Optional[torch.Tensor] = None

    def state_need(self) -> StateNeed:
        return StateNeed((self.width,), torch.float32)

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        w, d = self.width, self.dim
        return {
            "wz.weight": ExpectedTensor((w, d)), "wz.bias": ExpectedTensor((w,)),
            "wx.weight": ExpectedTensor((w, d)), "wx.bias": ExpectedTensor((w,)),
            "wg.weight": ExpectedTensor((w, d)), "wo.weight": ExpectedTensor((d, w)),
        }

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        f32 = dict(device=self.env.device, dtype=torch.float32)
        self.w_in = torch.cat([as_compute(tensors[n], self.env) for n in ("wz.weight", "wx.weight", "wg.weight")])   # rows [wz; wx; wg]
        self.b_in = torch.cat([tensors["wz.bias"].to(**f32), tensors["wx.bias"].to(**f32),
                               torch.zeros(self.width, **f32)]).contiguous()
        self.wo = as_compute(tensors["wo.weight"], self.env)

    def forward(self, x: torch.Tensor, ctx, cache) -> PendingProduct:
        ops = self.env.ops
        proj = ops.linear(x, self.w_in, partials_ok=True)
        y = ops.mingru_scan(proj, self.b_in, cache.state, ctx.q_start, ctx.state_slot, ctx.fresh,
                            n_seqs=ctx.n_seqs, max_q_len=ctx.max_q_len, out_dtype=self.env.dtype)
        return PendingProduct(y, self.wo)
