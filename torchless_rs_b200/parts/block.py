"""The arrangement of parts in a layer.  Pre-norm residual block:
h += mixer(norm1(h)); h += feed_forward(norm2(h)); the residual is the stream before
the norm (reference: src/model/modules/layer.rs:28-56).  The stream stays in 32-bit
and each part adds into it."""
from __future__ import annotations

import torch

from .registry import register_block
from .runtime import Runtime


@register_block("prenorm")
class PreNormBlock:
    """Interface of every block: a class attribute `norm_roles` (the norms this kind of block
    takes; a layer's spec must give exactly these), a constructor `(spec, rt, mixer,
    feed_forward, norms)` with `norms` a dictionary by role, the attributes `mixer`,
    `feed_forward` and `norms`, and `forward(x, batch)`, which updates the 32-bit stream `x`
    [tokens, hidden] in place.

    Optional, for blocks that let the products around a norm take it over: `takes_carry =
    True`, `first_norm` (the norm whose input the block before may prepare; None if its mixer
    cannot use one) and `forward(x, batch, carry, next_norm)` returning a carry for
    `next_norm` or None.  A block without `takes_carry` is called with `(x, batch)` only."""
    norm_roles = ("mixer_norm", "feed_forward_norm")
    takes_carry = True

    def __init__(self, spec, rt: Runtime, mixer, feed_forward, norms):
        self.rt = rt
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norms = dict(norms)
        self.mixer_norm = norms["mixer_norm"]
        self.feed_forward_norm = norms["feed_forward_norm"]

    @property
    def first_norm(self):
        return self.mixer_norm if getattr(self.mixer, "accepts_carry", False) else None

    def forward(self, x: torch.Tensor, batch, carry=None, next_norm=None):
        """`carry`: the input of this block's first norm if the product before it prepared
        it (else None).  `next_norm`: the norm that follows this block; the block returns
        a carry for it if its last product could prepare one (else None).

        A norm is folded into its neighbours only if it says it is `foldable` and both
        neighbours say they `accepts_carry`; otherwise the norm kernel runs."""
        from .linear import new_carry
        rt = self.rt
        xn = rt.workspace.get("block_normed", x.shape, rt.act_dtype)
        fold = not rt.is_f32

        def can_fold(norm, producer, consumer):
            return (fold and norm is not None and getattr(norm, "foldable", False)
                    and getattr(producer, "accepts_carry", False)
                    and getattr(consumer, "accepts_carry", False))

        inp = carry if (carry is not None and carry.valid) else self.mixer_norm(x, xn)
        c2 = None
        if can_fold(self.feed_forward_norm, self.mixer, self.feed_forward):
            c2 = new_carry(rt, "a", x.shape[0], self.feed_forward_norm.size, self.feed_forward_norm.eps)
            self.mixer.forward(inp, x, batch, emit=(self.feed_forward_norm.weight, c2))
        else:
            self.mixer.forward(inp, x, batch)
        inp2 = c2 if (c2 is not None and c2.valid) else self.feed_forward_norm(x, xn)
        c3 = None
        if next_norm is not None and getattr(next_norm, "foldable", False) and fold and \
                getattr(self.feed_forward, "accepts_carry", False):
            c3 = new_carry(rt, "b", x.shape[0], next_norm.size, next_norm.eps)
            self.feed_forward.forward(inp2, x, batch, emit=(next_norm.weight, c3))
        else:
            self.feed_forward.forward(inp2, x, batch)
        return c3 if (c3 is not None and c3.valid) else None


@register_block("prenorm_mixer_only")
class PreNormMixerBlock:
    """The pre-norm block of a layer without a feed-forward: x += mixer(norm1(x))."""
    norm_roles = ("mixer_norm",)

    def __init__(self, spec, rt: Runtime, mixer, feed_forward, norms):
        self.rt = rt
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norms = dict(norms)
        self.mixer_norm = norms["mixer_norm"]

    def forward(self, x: torch.Tensor, batch) -> None:
        rt = self.rt
        xn = rt.workspace.get("block_normed", x.shape, rt.act_dtype)
        self.mixer.forward(self.mixer_norm(x, xn), x, batch)


class StreamCopy:
    """What a branch-norm block hands to the next one: the stream in the activation type, as the
    kernel that last changed the stream wrote it.  (`valid` is False so that a block that expects the
    prepared input of a norm ignores it.)"""
    valid = False

    def __init__(self, xb: torch.Tensor):
        self.xb = xb


@register_block("branchnorm")
class BranchNormBlock:
    """x <- x + m * norm_1(mixer(x)); x <- x + m * norm_2(feed_forward(x)): the sublayers read the
    stream itself and the norm sits on each branch's output.  Parameter: `residual_mult` (m).

    The branch writes its output to a 32-bit buffer; one kernel takes its root mean square, adds
    m * gain * y / rms to the stream and writes the stream's copy in the activation type, which the next
    sublayer's products read (in 32-bit the stream is that copy).  A sublayer that says
    `can_overwrite` stores its output (`forward(..., overwrite=True)`); any other adds into the zeroed
    buffer, so every registered mixer and feed-forward fits.  Norms: any with a single `gain`, or
    with a `weight` per coordinate."""
    norm_roles = ("mixer_out_norm", "feed_forward_out_norm")
    takes_carry = True
    first_norm = None   # no norm stands before this block's first product

    def __init__(self, spec, rt: Runtime, mixer, feed_forward, norms):
        self.rt = rt
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norms = dict(norms)
        self.mult = float(spec.get("residual_mult", 1.0))
        self._gains = {}

    def _gain(self, norm):
        g = getattr(norm, "gain", None)
        if g is not None:
            return g
        key = id(norm)
        if key not in self._gains:
            self._gains[key] = norm.weight.to(torch.float32).contiguous()
        return self._gains[key]

    def _branch(self, part, norm, x, xb, batch):
        rt = self.rt
        y = rt.workspace.get("branch_out", x.shape, torch.float32)
        if getattr(part, "can_overwrite", False):
            part.forward(xb, y, batch, overwrite=True)
        else:
            y.zero_()
            part.forward(xb, y, batch)
        gain = self._gain(norm)
        if gain.numel() != 1:
            # a weight per coordinate: the norm's own kernel, then the scaled sum
            yn = rt.workspace.get("branch_normed", x.shape, rt.act_dtype)
            norm(y, yn)
            x.add_(yn.to(torch.float32), alpha=self.mult)
            if xb is not x:
                xb.copy_(x)
            return
        rt.ops.branch_norm_add(y, gain, self.mult, norm.eps, x, None if xb is x else xb)

    def forward(self, x: torch.Tensor, batch, carry=None, next_norm=None):
        rt = self.rt
        if rt.is_f32:
            xb = x
        elif isinstance(carry, StreamCopy) and carry.xb.shape == x.shape:
            xb = carry.xb
        else:
            xb = rt.workspace.get("branch_in", x.shape, rt.act_dtype)
            rt.ops.convert_into(x, xb)
        self._branch(self.mixer, self.norms["mixer_out_norm"], x, xb, batch)
        if "feed_forward_out_norm" in self.norms:
            self._branch(self.feed_forward, self.norms["feed_forward_out_norm"], x, xb, batch)
        return None if xb is x else StreamCopy(xb)


@register_block("branchnorm_mixer_only")
class BranchNormMixerBlock(BranchNormBlock):
    """The same block for a layer without a feed-forward: x <- x + m * norm_1(mixer(x))."""
    norm_roles = ("mixer_out_norm",)


class NormedInput:
    """What a sandwich block hands to the next one: the next block's first norm already applied to the
    stream, written by the kernel that last changed the stream.  (`valid` is False so that a block that
    expects the prepared input of a folded norm ignores it.)"""
    valid = False

    def __init__(self, xn: torch.Tensor, norm):
        self.xn, self.norm = xn, norm


@register_block("sandwich")
class SandwichBlock:
    """x <- x + N_1b(mixer(N_1(x))); x <- x + N_2b(feed_forward(N_2(x))): a norm before and after every
    sublayer, each with its own weight.

    A sublayer writes its output to a 32-bit buffer (one that says `can_overwrite` stores it, any other adds
    into the zeroed buffer, so every registered mixer and feed-forward fits); one kernel norms that output,
    adds it to the stream and applies the norm that comes next (this block's second, or the next block's
    first, which is handed on as a `NormedInput`), so the stream crosses memory once per sublayer.  The
    fused kernel takes norms with a plain weight per coordinate (`weight`, `eps`); the next norm is fused
    only if its weight has the same type as this one's."""
    norm_roles = ("mixer_norm", "mixer_out_norm", "feed_forward_norm", "feed_forward_out_norm")
    takes_carry = True

    def __init__(self, spec, rt: Runtime, mixer, feed_forward, norms):
        self.rt = rt
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norms = dict(norms)

    @property
    def first_norm(self):
        return self.norms["mixer_norm"]

    def _sublayer(self, part, norm_in, norm_out, x, xn, batch, next_norm):
        """x += norm_out(part(xn)); returns next_norm(x) if it could be taken along, else None."""
        rt = self.rt
        y = rt.workspace.get("branch_out", x.shape, torch.float32)
        if getattr(part, "can_overwrite", False):
            part.forward(xn, y, batch, overwrite=True)
        else:
            y.zero_()
            part.forward(xn, y, batch)
        fuse = (next_norm is not None and getattr(next_norm, "weight", None) is not None
                and getattr(next_norm, "size", None) == x.shape[1]
                and next_norm.weight.dtype == norm_out.weight.dtype)
        if not fuse:
            rt.ops.norm_add_norm(y, norm_out.weight, norm_out.eps, x)
            return None
        out = rt.workspace.get("block_normed", x.shape, rt.act_dtype)
        rt.ops.norm_add_norm(y, norm_out.weight, norm_out.eps, x, next_norm.weight, next_norm.eps, out)
        return out

    def _input(self, norm, x, carry):
        if isinstance(carry, NormedInput) and carry.norm is norm and carry.xn.shape == x.shape:
            return carry.xn
        return norm(x, self.rt.workspace.get("block_normed", x.shape, self.rt.act_dtype))

    def forward(self, x: torch.Tensor, batch, carry=None, next_norm=None):
        n = self.norms
        xn = self._input(n["mixer_norm"], x, carry)
        second = n.get("feed_forward_norm")
        got = self._sublayer(self.mixer, n["mixer_norm"], n["mixer_out_norm"], x, xn, batch,
                             second if second is not None else next_norm)
        if second is None:
            return NormedInput(got, next_norm) if got is not None else None
        xn = got if got is not None else second(x, self.rt.workspace.get("block_normed", x.shape, self.rt.act_dtype))
        got = self._sublayer(self.feed_forward, second, n["feed_forward_out_norm"], x, xn, batch, next_norm)
        return NormedInput(got, next_norm) if got is not None else None


@register_block("sandwich_mixer_only")
class SandwichMixerBlock(SandwichBlock):
    """The same block for a layer without a feed-forward: x <- x + N_1b(mixer(N_1(x)))."""
    norm_roles = ("mixer_norm", "mixer_out_norm")
