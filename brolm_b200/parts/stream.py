"""Parts that act on the residual stream itself, between two layers."""
from __future__ import annotations

import torch

from .. import kernels
from .base import ParamSpec, Part, register_part
from .linear import linear


class ConcatLinear(Part):
    """h <- W [h; h0]: the stream and the embedding's output side by side through one matrix
    (hidden, 2 hidden), h's columns first.  A model that runs a span of layers several times with the
    same weights puts this in front of every pass, so each pass sees the tokens again.  The product takes
    the step's element type with float accumulation; the new stream is float."""

    kind = "stream"
    graph_safe = True

    def __init__(self, hidden: int):
        self.hidden = hidden

    def param_specs(self):
        return {"weight": ParamSpec((self.hidden, 2 * self.hidden))}

    def forward(self, h: torch.Tensor, h0: torch.Tensor, ctx) -> torch.Tensor:
        both = torch.empty((h.shape[0], 2 * self.hidden), dtype=ctx.dtype, device=h.device)
        kernels.concat_cast(h, h0, both)
        out = linear(both, self.params["weight"], out_dtype=torch.float32)
        return out


register_part("stream", "concat_linear", ConcatLinear)
