"""Recurrent mixers: a state of fixed size per request, in a slot of the cache manager."""
import torch

from ..cache.needs import CacheNeed
from ..csrc import ops
from .base import Part
from .linear import Linear
from .plan import WeightDecl
from .registry import register_part


@register_part("mixer", "min_gru")
class MinGRU(Part):
    """A gated recurrence whose gates read the current token only:
    z = sigmoid(h·Wzᵀ + bz), u = h·Wxᵀ + bx, candidate c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0);
    S_t = (1 - z) S_(t-1) + z c, element by element; out = (S_t * silu(h·Wgᵀ))·Woᵀ.
    The three input projections are one product whose 32-bit result the scan kernel reads;
    gates, candidate and state are 32-bit; the state (`width` floats) starts at zero and is
    carried per request.  params: size, width."""

    @classmethod
    def declare_weights(cls, params):
        E, W = params["size"], params["width"]
        return {"gate_weight": WeightDecl((W, E), "matrix"), "gate_bias": WeightDecl((W,), "bias"),
                "cand_weight": WeightDecl((W, E), "matrix"), "cand_bias": WeightDecl((W,), "bias"),
                "out_gate_weight": WeightDecl((W, E), "matrix"),
                "out_weight": WeightDecl((E, W), "residual_matrix")}

    def load(self, tensors, store):
        W = self.params["width"]
        names = [tensors[k] for k in ("gate_weight", "cand_weight", "out_gate_weight")]
        w = store.computed("+".join(r.name for r in names), lambda: torch.cat([r.tensor.float() for r in names], 0))
        bz, bx = tensors["gate_bias"], tensors["cand_bias"]
        b = store.computed(bz.name + "+" + bx.name + "+0", kind="vector",
                           make=lambda: torch.cat([bz.tensor.float(), bx.tensor.float(), torch.zeros(W)]))
        self.inp = Linear(w, b)
        self.out = Linear(store.matrix(tensors["out_weight"]), None)

    def cache_need(self):
        return CacheNeed.state((self.params["width"],), "float32")

    def workspace_per_token(self):
        act = 4 if self.rt.dtype == "float32" else 2
        # the projections, the gated state, and (steps with long portions) the chunk sums: two
        # floats a channel for every chunk's worth of tokens and three for every request, of
        # which a step has no more than tokens
        W = self.params["width"]
        return W * (12 + act) + 12 * W + 8 * W // ops.GATED_SCAN_PIECE + 8

    def forward(self, ctx, h, residual, cache, position=None, out=None):
        T, W = h.shape[0], self.params["width"]
        pre = ctx.alloc((T, 3 * W), torch.float32)
        self.inp.forward(ctx, h, out=pre)
        y = ctx.alloc((T, W), self.rt.act_dtype)
        need = ops.mingru_scan_workspace(ctx.R, W, T, ctx.max_q_len)
        ws = ctx.alloc((need,), torch.float32) if need else None
        ops.mingru_scan(ctx.columns(pre, 0, W), ctx.columns(pre, W, 2 * W), ctx.columns(pre, 2 * W, 3 * W), y,
                        cache.tensor, ctx.q_start, ctx.state_slots, ctx.R, ctx.max_q_len, workspace=ws)
        return self.out.forward(ctx, y, out=out, residual=residual)
