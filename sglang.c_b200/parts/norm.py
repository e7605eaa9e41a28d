"""Normalisation parts."""
from ..csrc import ops
from .base import Part
from .plan import WeightDecl
from .registry import register_part


@register_part("norm", "layer_norm")
class LayerNorm(Part):
    """y = (x-mean)/sqrt(var+eps)*weight + bias over the last axis, biased
    variance, statistics in 32-bit (reference src/ops.c:199-218).
    params: size, eps, bias (default true; false: a gain only), groups (default 1: the row is
    split into so many equal consecutive parts, each with statistics of its own; gain and bias
    span the row)."""

    form = "layer"

    @classmethod
    def declare_weights(cls, params):
        d = {"weight": WeightDecl((params["size"],), "norm_gain")}
        if params.get("bias", True):
            d["bias"] = WeightDecl((params["size"],), "norm_bias")
        return d

    def load(self, tensors, store):
        ref = tensors["weight"]
        if self.params.get("one_plus"):
            # a gain stored around zero: the kernels multiply by 1 + w, formed once
            self.weight = store.computed(ref.name + "+1", kind="vector", make=lambda: ref.tensor.float() + 1.0)
        else:
            self.weight = store.vector(ref)
        self.bias = store.vector(tensors["bias"]) if "bias" in tensors else None

    @property
    def groups(self):
        return int(self.params.get("groups", 1))

    def forward(self, ctx, x, out, rows=None):
        if self.bias is not None and self.form == "layer" and self.groups == 1:
            ops.layernorm(x, self.weight, self.bias, float(self.params["eps"]), out, rows=rows)
        else:
            src = x[:out.shape[0]] if rows is None else x
            ops.norm_rows(src, self.weight, self.bias, float(self.params["eps"]), out, form=self.form,
                          src_rows=rows, groups=self.groups)
        return out

    def add_into(self, ctx, y, residual, mix=None, then=None, then_cast=None):
        """residual += norm(y): the norm behind a sublayer, summed into the 32-bit stream.  In the
        same launch, if asked: `mix` = (hist, n_terms, weights), the depth mix of the summed rows
        (see ops.depth_mix), and `then` = (norm part, out): out = that norm of the rows as they
        then are (the norm ahead of the next sublayer).  Returns which of the two it did: a norm
        with a bias, or a source that is not 32-bit, leaves them to the caller.
        `then_cast` (instead of `then`): a buffer that takes the summed rows in its own precision,
        for a next sublayer that reads the stream itself; always done (in the same launch where the
        fused kernel serves, by a second one else)."""
        if then_cast is not None:
            if self.groups == 1 and self.bias is None and y.dtype == residual.dtype \
                    and y.shape[0] == residual.shape[0] and residual.is_contiguous():
                ops.norm_add_tail(y, self.weight, float(self.params["eps"]), residual, form=self.form,
                                  then=(None, 0.0, "copy", then_cast))
            else:
                ops.norm_rows(y, self.weight, self.bias, float(self.params["eps"]), residual[:y.shape[0]],
                              form=self.form, add=True, groups=self.groups)
                ops.cast_rows(residual[:y.shape[0]], then_cast)
            return True
        fused = self.groups == 1 and (then is None or then[0].groups == 1) \
            and y.dtype == residual.dtype and self.bias is None and (then is None or then[0].bias is None) \
            and y.shape[0] == residual.shape[0] and residual.is_contiguous() and (mix is not None or then is not None)
        if not fused:
            ops.norm_rows(y, self.weight, self.bias, float(self.params["eps"]), residual[:y.shape[0]],
                          form=self.form, add=True, groups=self.groups)
            return False
        nxt = None if then is None else (then[0].weight, float(then[0].params["eps"]), then[0].form, then[1])
        ops.norm_add_tail(y, self.weight, float(self.params["eps"]), residual, form=self.form, mix=mix, then=nxt)
        return True

    def scatter(self, ctx, y, dst, dst_rows):
        """dst[dst_rows[r], :] = norm(y[r, :]): normalised rows straight into a cache's rows."""
        ops.norm_rows(y, self.weight, self.bias, float(self.params["eps"]), dst, form=self.form,
                      dst_rows=dst_rows, groups=self.groups)
        return dst


@register_part("norm", "rms_norm")
class RMSNorm(LayerNorm):
    """y = x / sqrt(mean(x^2) + eps) * weight, eps inside the root, statistics in 32-bit.
    params: size, eps, groups (default 1; more: each of so many equal consecutive parts of the row is
    divided by its own root mean square), one_plus (default false; true: the file's tensor is stored
    around zero and the gain is 1 + it)."""

    form = "rms"

    @classmethod
    def declare_weights(cls, params):
        return {"weight": WeightDecl((params["size"],), "norm_gain")}
