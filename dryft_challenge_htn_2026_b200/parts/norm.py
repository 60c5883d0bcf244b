"""RMSNorm (reference: engine/engine.py:107-110, engine/fused.py:152-172)."""
import torch

from ..config.specs import GroupRMSNormSpec, OnePlusRMSNormSpec, RMSNormSpec, ScalarRMSNormSpec
from ..csrc import api
from .base import ParamDecl, Part, register_part


class NormedDelta:
    """A sublayer's output that still has to go through a norm of its own before it joins the residual stream:
    ``delta`` (a tensor or a ``csrc.api.Partial``) and ``norm`` (an ``RMSNorm`` part). The norm that follows the sum
    takes it as its ``delta`` and does both in one kernel."""

    def __init__(self, delta, norm):
        self.delta, self.norm = delta, norm

    def to_float32(self):
        """What joins the stream, worked out plainly (for dumps of the stream between layers)."""
        d = self.delta.ws.sum(0) if isinstance(self.delta, api.Partial) else self.delta.to(torch.float32)
        return d * torch.rsqrt((d * d).mean(-1, keepdim=True) + self.norm.spec.eps) * self.norm.weight


class RMSNorm(Part):
    """y = w * x * rsqrt(mean(x^2) + eps), statistics in float32, weight held in float32."""
    takes_partial = True     # add_forward adds up split-K partial sums (csrc.api.Partial) while it reads them

    def param_decls(self):
        return [ParamDecl(self.spec.tensor, (self.spec.dim,), init="norm", keep_float32=True)]

    def bind(self, tensors):
        self.weight = tensors[self.spec.tensor].to(torch.float32).contiguous()

    def add_forward(self, h, delta, out, rows=None):
        """h (float32 residual stream) += delta (a tensor, a ``csrc.api.Partial`` or None; a ``NormedDelta`` goes
        through its own norm first); out = norm(h). ``rows``: only these rows, into out[0..len(rows)), leaving h as
        it is."""
        if isinstance(delta, NormedDelta):
            api.normed_add_rmsnorm(h, delta.delta, delta.norm.weight, delta.norm.spec.eps, self.weight, self.spec.eps, out, rows)
        else:
            api.add_rmsnorm(h, delta, self.weight, self.spec.eps, out, rows)
        return out

    def scale_add_forward(self, h, alpha, delta, out):
        """The norm after the sum: h = norm(alpha * h + delta), written back to the float32 stream; out = the
        same in the storage type. ``delta`` a tensor or a ``csrc.api.Partial``."""
        api.scale_add_rmsnorm(h, alpha, delta, self.weight, self.spec.eps, out)
        return out


register_part(RMSNormSpec, RMSNorm)


class ScalarRMSNorm(RMSNorm):
    """RMS norm with one learned number for all coordinates: y = g * x * rsqrt(mean(x^2) + eps). The
    number is spread over the width when it is bound, so the norm runs on the kernels of ``RMSNorm``
    (fused with the residual add, with the embedding, gathered at the wanted rows). Its tensor has no
    name of its own under the part's prefix: the prefix is the tensor's name."""

    def param_decls(self):
        return [ParamDecl("", (), init="norm", keep_float32=True)]

    def bind(self, tensors):
        self.gain = tensors[""].to(torch.float32).reshape(())
        self.weight = self.gain.expand(self.spec.dim).contiguous()


register_part(ScalarRMSNormSpec, ScalarRMSNorm)


class OnePlusRMSNorm(RMSNorm):
    """RMS norm whose stored weight sits around zero: y = (1 + w) * x * rsqrt(mean(x^2) + eps). One is added in
    float32 when the tensor is bound, so the norm runs on the kernels of ``RMSNorm``. Like the scalar norm its
    tensor is named by the part's prefix itself."""

    def param_decls(self):
        return [ParamDecl("", (self.spec.dim,), init="around_zero", keep_float32=True)]

    def bind(self, tensors):
        self.weight = (1.0 + tensors[""].to(torch.float32)).contiguous()


register_part(OnePlusRMSNormSpec, OnePlusRMSNorm)


class GroupRMSNorm(Part):
    """RMS norm in groups: the row in ``groups`` equal consecutive parts, each over its own root mean square, the whole
    times a weight of the row's size. Statistics in float32, weight held in float32; one kernel with the residual add,
    also gathered at the wanted rows (so it can stand as first, inner and final norm)."""
    takes_partial = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        if spec.groups < 1 or spec.dim % spec.groups:
            raise ValueError(f"a norm in {spec.groups} parts of {spec.dim} coordinates")

    def param_decls(self):
        return [ParamDecl(self.spec.tensor, (self.spec.dim,), init="norm", keep_float32=True)]

    def bind(self, tensors):
        self.weight = tensors[self.spec.tensor].to(torch.float32).contiguous()

    def add_forward(self, h, delta, out, rows=None):
        api.add_group_rmsnorm(h, delta, self.weight, self.spec.eps, self.spec.groups, out, rows)
        return out


register_part(GroupRMSNormSpec, GroupRMSNorm)
