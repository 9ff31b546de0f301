"""Parts that mix the residual streams of several depths."""
import torch

from ..csrc import ops
from .base import Part
from .plan import WeightDecl
from .registry import register_part


@register_part("stream_mix", "depth_weighted_average")
class DepthWeightedAverage(Part):
    """With X_0 the embedding output and X_(i+1) the result of layer i, what leaves layer i is
    sum_{j=0..i+1} w[j] * X_j, w being this layer's own i+2 weights.  The X_j of the step's
    tokens are kept, 32-bit, in one buffer of the step workspace that the first layer takes
    (`begin`, ahead of the block's own buffers) and every layer adds to (`finish`).
    params: index (i), n_layers, size."""

    @classmethod
    def declare_weights(cls, params):
        return {"weights": WeightDecl((params["index"] + 2,), "norm_gain")}

    def load(self, tensors, store):
        self.weights = store.vector(tensors["weights"])

    def workspace_per_token(self):
        return 4 * self.params["size"] * (self.params["n_layers"] + 1)

    def begin(self, ctx, x):
        if self.params["index"] == 0:
            hist = ctx.alloc((self.params["n_layers"] + 1,) + tuple(x.shape), torch.float32)
            ctx.shared["depth_streams"] = hist
            ops.depth_mix(x, hist, 1, None)

    def terms(self, ctx):
        """(streams kept so far, terms of this layer's sum, its weights): for a kernel that does
        the mix itself, in place of finish()."""
        return ctx.shared["depth_streams"], self.params["index"] + 2, self.weights

    def finish(self, ctx, x):
        ops.depth_mix(x, ctx.shared["depth_streams"], self.params["index"] + 2, self.weights)
        return x
