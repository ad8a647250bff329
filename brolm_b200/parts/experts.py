"""Routed experts: a feed-forward made of many small ones, of which a token uses a few."""
from __future__ import annotations

import torch

from .. import kernels
from .base import ParamSpec, Part, register_part
from .linear import linear


class RoutedExperts(Part):
    """y = sum over the token's ``top`` experts e of  W_down[e] act(W_up[e] (g_e x)),  no biases.

    Router: z = W_r x summed in float (by the router kernel in one fixed order; for a prompt in bfloat16 by a
    matrix product with float accumulation); the ``top`` largest z are chosen; g_e = logistic(z_e), not
    renormalised.  With ``scale_input`` the gate multiplies the expert's input (one rounding to the step's
    element type), not its output.  ``activation``: "relu2" (the square of relu) or "none".

    On the device: route -> sort the (token, choice) pairs by expert -> one grouped product per matrix over
    tiles of each expert's pairs -> float results [top, tokens, hidden], which the residual kernel
    adds in the order of the choices.  Nothing is read back to the host.  With many pairs per expert (a
    prompt) the products run on tcgen05 over 128-row tiles, the tokens' rows first copied into expert order;
    with few (decoding) on mma.sync over 64-row tiles, as a stream of the chosen experts' matrices.
    """

    kind = "feedforward"
    graph_safe = True
    ROUTER_PRODUCT_ROWS = 256      # from this many tokens on the router's scores are a matrix product

    def __init__(self, hidden: int, inter: int, experts: int, top: int, activation: str = "relu2",
                 scale_input: bool = True):
        if not 1 <= top <= experts:
            raise ValueError("routed experts: 1 <= top <= experts")
        if activation not in kernels.EXPERT_ACTS:
            raise ValueError(f"routed experts: unknown activation '{activation}'")
        if not scale_input:
            raise ValueError("routed experts: a gate on the expert's output is not built")
        self.hidden, self.inter, self.experts, self.top, self.activation = hidden, inter, experts, top, activation

    def param_specs(self):
        specs = {"router": ParamSpec((self.experts, self.hidden))}
        for e in range(self.experts):
            specs[f"e{e}.up"] = ParamSpec((self.inter, self.hidden))
            specs[f"e{e}.down"] = ParamSpec((self.hidden, self.inter))
        return specs

    def bind(self, params):
        self.router = params["router"]
        kinds = {params[f"e{e}.{n}"].dtype for e in range(self.experts) for n in ("up", "down")} | {self.router.dtype}
        if len(kinds) > 1:
            raise TypeError("routed experts: the experts' matrices and the router must have one element type")
        self.w_up = torch.stack([params[f"e{e}.up"] for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([params[f"e{e}.down"] for e in range(self.experts)]).contiguous()
        self.params = {}

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        """x (tokens, hidden) -> [top, tokens, hidden] float32 partial results."""
        T, dev = x.shape[0], x.device
        if x.dtype != self.router.dtype:
            x = x.to(self.router.dtype)
        pairs = T * self.top
        ids = torch.empty((T, self.top), dtype=torch.int32, device=dev)
        gates = torch.empty((T, self.top), dtype=torch.float32, device=dev)
        if x.dtype == torch.bfloat16 and T >= self.ROUTER_PRODUCT_ROWS and self.experts <= 1024 and self.hidden % 8 == 0:
            # a prompt: the scores as one matrix product (bfloat16 products are exact in float, the sums are
            # float), then the choice; the router kernel's float multiply-adds are what bounds it from here on
            kernels.route_pick(linear(x, self.router, out_dtype=torch.float32), self.top, ids, gates)
        else:
            kernels.route_topk(x, self.router, self.top, ids, gates)
        perm = torch.empty(pairs, dtype=torch.int32, device=dev)
        offsets = torch.empty(self.experts + 1, dtype=torch.int32, device=dev)
        u = torch.empty((pairs, self.inter), dtype=x.dtype, device=dev)
        if kernels.experts_tc_ok(x, self.w_up, self.w_down, pairs):
            rows = kernels.GROUP_ROWS_TC
            tiles = torch.empty((2, kernels.group_tiles(pairs, self.experts, rows)), dtype=torch.int32, device=dev)
            kernels.group_pairs(ids, self.experts, perm, offsets, tiles, rows)
            xs = torch.empty((pairs, self.hidden), dtype=x.dtype, device=dev)
            kernels.gather_rows(x, perm, self.top, xs)
            kernels.experts_linear_tc(xs, self.w_up, u, perm, offsets, tiles, self.top, T, scale=gates,
                                      activation=self.activation)
            y = torch.empty((self.top, T, self.hidden), dtype=torch.float32, device=dev)
            kernels.experts_linear_tc(u, self.w_down, y, perm, offsets, tiles, self.top, T, down=True)
            return y
        tiles = torch.empty((2, kernels.group_tiles(pairs, self.experts)), dtype=torch.int32, device=dev)
        kernels.group_pairs(ids, self.experts, perm, offsets, tiles)
        kernels.experts_linear(x, self.w_up, u, perm, offsets, tiles, self.top, T, scale=gates,
                               activation=self.activation)
        y = torch.empty((self.top, T, self.hidden), dtype=torch.float32, device=dev)
        kernels.experts_linear(u, self.w_down, y, perm, offsets, tiles, self.top, T, down=True)
        return y


register_part("feedforward", "routed_experts", RoutedExperts)
