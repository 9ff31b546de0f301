"""Feed-forward parts."""
import torch

from .base import Part
from .linear import Linear, declare_linear
from .plan import WeightDecl
from .registry import register_part


@register_part("feed_forward", "mlp")
class MLP(Part):
    """residual += act(h·W_up + b_up)·W_down + b_down
    (reference src/gpt2.c:283-292; activation src/ops.c:233-241).
    params: size, inner_size, activation ("gelu_tanh" | "gelu_erf" | "xielu"), bias,
    weight_layout ("conv1d" = [in,out] in the file, "linear" = [out,in]).
    "xielu" carries two numbers (p, q) of its own in a tensor `act_params`:
    act(z) = softplus(p) z^2 + z/2 for z > 0, (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2 otherwise."""

    @classmethod
    def declare_weights(cls, params):
        lay, bias = params.get("weight_layout", "linear"), params.get("bias", True)
        up = declare_linear(params["size"], params["inner_size"], lay, bias)
        down = declare_linear(params["inner_size"], params["size"], lay, bias, init="residual_matrix")
        d = {"up_" + k: v for k, v in up.items()}
        d.update({"down_" + k: v for k, v in down.items()})
        if params["activation"] == "xielu":
            d["act_params"] = WeightDecl((2,), "bias")
        return d

    def load(self, tensors, store):
        lay = self.params.get("weight_layout", "linear")
        self.up = Linear.from_refs(store, tensors["up_weight"], tensors.get("up_bias"), lay)
        self.down = Linear.from_refs(store, tensors["down_weight"], tensors.get("down_bias"), lay)
        self.act_params = self.act_slot = None
        if self.params["activation"] == "xielu":
            from ..csrc import ops
            import math
            p, q = (float(v) for v in tensors["act_params"].tensor.double().tolist())
            softplus = lambda v: max(v, 0.0) + math.log1p(math.exp(-abs(v)))
            self.act_params = (softplus(p), 0.5 + softplus(q))
            if self.rt is not None:
                libs = ["gemm_simt"] + (["gemm_tc", "gemm_few"] if self.rt.dtype == "bfloat16" else [])
                self.act_slot = ops.register_act_params(*self.act_params, libs)

    act_params = act_slot = None

    def workspace_per_token(self):
        act = 4 if self.rt.dtype == "float32" else 2
        return (act + (4 if self.params["activation"] == "xielu" else 0)) * self.params["inner_size"]

    def act_in_own_kernel(self):
        """An activation with numbers of its own is applied in the up-projection's epilogue from a
        slot of the kernel libraries' parameter tables; only a model with more such activations
        than slots sends the product's 32-bit result through a kernel of the activation."""
        return self.params["activation"] == "xielu" and self.act_slot is None

    def forward(self, ctx, h, residual, out=None):
        from ..csrc import ops
        T = h.shape[0]
        u = ctx.alloc((T, self.params["inner_size"]), self.rt.act_dtype)
        if self.act_in_own_kernel():
            z = ctx.alloc((T, self.params["inner_size"]), torch.float32)
            self.up.forward(ctx, h, out=z)
            ops.xielu(z, u, *self.act_params)
        elif self.act_slot is not None:
            self.up.forward(ctx, h, out=u, act=(self.params["activation"], self.act_slot))
        else:
            self.up.forward(ctx, h, out=u, act=self.params["activation"])
        return self.down.forward(ctx, u, out=out, residual=residual)
