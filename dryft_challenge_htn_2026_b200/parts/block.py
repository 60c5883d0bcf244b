"""Pre-norm residual block: h += mixer(norm_in(h)); h += feed_forward(norm_post(h)).

The residual stream ``h`` is float32. Each add is fused with the norm that follows it, so the
block takes the previous block's not-yet-added output as ``pending`` and returns its own
feed-forward output the same way (the reference fuses the same pair: engine/engine.py:493-495).
A mixer or feed-forward may return its output as split-K partial sums (``csrc.api.Partial``); a
norm that says ``takes_partial`` adds them up while it reads, for any other they are summed first.
"""
import torch

from ..config.specs import LayerSpec, PostNormLayerSpec, SandwichLayerSpec
from ..csrc import api
from .base import ParamDecl, Part, build_part, register_part
from .norm import NormedDelta, RMSNorm


class PreNormBlock(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.norm_in = build_part(spec.norm_in, rt)
        self.mixer = build_part(spec.mixer, rt)
        # a layer may go without a feed-forward: then the mixer's output is what it hands on
        self.norm_post = build_part(spec.norm_post, rt) if spec.feed_forward is not None else None
        self.feed_forward = build_part(spec.feed_forward, rt) if spec.feed_forward is not None else None

    def _subparts(self):
        return [(getattr(self, attr), pre) for attr, pre in self.spec.names if getattr(self, attr) is not None]

    def param_decls(self):
        return [ParamDecl(pre + p.name, p.shape, p.init, p.keep_float32) for part, pre in self._subparts()
                for p in part.param_decls()]

    def bind(self, tensors):
        for part, pre in self._subparts():
            part.bind({k[len(pre):]: v for k, v in tensors.items() if k.startswith(pre)})

    def step_weights(self):
        """The tensors a step streams once, whatever the batch (for the bytes a decode step must read)."""
        return [w for part, _ in self._subparts() for w in part.step_weights()]

    def step_plans(self):
        return [p for part, _ in self._subparts() for p in part.step_plans()]

    def cache_requests(self):
        return self.mixer.cache_requests()

    def prepare(self, max_positions):
        for part, _ in self._subparts():
            part.prepare(max_positions)

    def forward(self, ctx, h, pending, views, writes=True, a=None):
        """``a``: norm_in(h) if the caller already has it (the embedding kernel makes it for the
        first block). Returns the feed-forward output, still to be added to h."""
        if a is None:
            a = add_norm(self.norm_in, h, pending, self.rt.dtype)
        d = self.mixer.forward(ctx, views, a, writes)
        if self.feed_forward is None:
            return d
        a = add_norm(self.norm_post, h, d, self.rt.dtype)
        return self.feed_forward.forward(ctx, a)


def add_norm(norm, h, delta, dtype, rows=None):
    """h += delta, then norm(h) (of the rows ``rows`` only, leaving h alone, when given)."""
    if isinstance(delta, NormedDelta) and not isinstance(norm, RMSNorm):
        raise TypeError(f"{type(norm).__name__} cannot follow a sublayer whose output has a norm of its own")
    if isinstance(delta, api.Partial) and not getattr(norm, "takes_partial", False):
        delta = delta.sum(dtype)
    n = h.shape[0] if rows is None else rows.numel()
    out = torch.empty((n, h.shape[1]), dtype=dtype, device=h.device)
    return norm.add_forward(h, delta, out, rows)


register_part(LayerSpec, PreNormBlock)


class PostNormBlock(Part):
    """Norm after the sum: x <- norm_mix(alpha * x + mixer(x)), then x <- norm_ff(alpha * x + feed_forward(x)).
    The residual stream stays float32; each norm kernel writes the stream back and leaves its copy in the
    storage type, which is what the next sublayer (of this block or the next) reads: it travels as
    ``ctx.stream_copy``. Nothing is left pending for the block after it."""
    reads_stream = True      # the block's first sublayer reads the stream itself, not a norm of it

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.mixer = build_part(spec.mixer, rt)
        self.norm_mix = build_part(spec.norm_mix, rt)
        self.feed_forward = build_part(spec.feed_forward, rt) if spec.feed_forward is not None else None
        self.norm_ff = build_part(spec.norm_ff, rt) if spec.feed_forward is not None else None
        for n in (self.norm_mix, self.norm_ff):
            if n is not None and not hasattr(n, "scale_add_forward"):
                raise TypeError(f"{type(n).__name__} cannot stand after a sum: it has no scale_add_forward()")

    _subparts = PreNormBlock._subparts
    param_decls = PreNormBlock.param_decls
    bind = PreNormBlock.bind
    step_weights = PreNormBlock.step_weights
    step_plans = PreNormBlock.step_plans
    cache_requests = PreNormBlock.cache_requests
    prepare = PreNormBlock.prepare

    def forward(self, ctx, h, pending, views, writes=True, a=None):
        dtype = self.rt.dtype
        if pending is not None:          # a block before this one left its output to be added
            if isinstance(pending, NormedDelta):
                pending = pending.to_float32()
            if isinstance(pending, api.Partial):
                pending = pending.sum(dtype)
            api.stream_add(h, pending.to(torch.float32))
            ctx.stream_copy = None
        if a is None:
            a = getattr(ctx, "stream_copy", None)
        if a is None:
            a = torch.empty(h.shape, dtype=dtype, device=h.device)
            api.cast_rows(h, a)
        d = self.mixer.forward(ctx, views, a, writes)
        a = self.norm_mix.scale_add_forward(h, self.spec.alpha, d, torch.empty(h.shape, dtype=dtype, device=h.device))
        if self.feed_forward is not None:
            d = self.feed_forward.forward(ctx, a)
            a = self.norm_ff.scale_add_forward(h, self.spec.alpha, d, torch.empty(h.shape, dtype=dtype, device=h.device))
        ctx.stream_copy = a
        return None


register_part(PostNormLayerSpec, PostNormBlock)


class SandwichBlock(PreNormBlock):
    """A norm before and after each sublayer: h += norm_mix_out(mixer(norm_in(h))); h += norm_ff_out(feed_forward(
    norm_post(h))). Like the pre-norm block it takes the block before's output as ``pending`` and hands its own on, as
    a ``NormedDelta``: the norm of a sublayer's output, the sum and the norm behind the sum are one kernel."""

    def __init__(self, spec, rt):
        Part.__init__(self, spec, rt)
        self.norm_in = build_part(spec.norm_in, rt)
        self.mixer = build_part(spec.mixer, rt)
        self.norm_mix_out = build_part(spec.norm_mix_out, rt)
        has_ff = spec.feed_forward is not None
        self.norm_post = build_part(spec.norm_post, rt) if has_ff else None
        self.feed_forward = build_part(spec.feed_forward, rt) if has_ff else None
        self.norm_ff_out = build_part(spec.norm_ff_out, rt) if has_ff else None
        for n in (self.norm_in, self.norm_mix_out, self.norm_post, self.norm_ff_out):
            if n is not None and not isinstance(n, RMSNorm):
                raise TypeError(f"{type(n).__name__}: the norms around a sublayer run on the RMS norm's kernels")

    def forward(self, ctx, h, pending, views, writes=True, a=None):
        if a is None:
            a = add_norm(self.norm_in, h, pending, self.rt.dtype)
        d = NormedDelta(self.mixer.forward(ctx, views, a, writes), self.norm_mix_out)
        if self.feed_forward is None:
            return d
        a = add_norm(self.norm_post, h, d, self.rt.dtype)
        return NormedDelta(self.feed_forward.forward(ctx, a), self.norm_ff_out)


register_part(SandwichLayerSpec, SandwichBlock)
