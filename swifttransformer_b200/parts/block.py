"""Blocks: how a mixer, a feed-forward and norms are arranged around the
residual stream.

pre_norm  (OPT with do_layer_norm_before; src/csrc/model/gpt/gpt.cc:304-503):
    r = x + mixer(norm1(x));  x' = r + ffn(norm2(r))
post_norm (do_layer_norm_before false; the reference refuses it, gpt.cc:238-240):
    r = norm1(x + mixer(x));  x' = norm2(r + ffn(r))
norm_after (the norm on the sub-layer's output only; the sub-layers read x itself):
    r = x + mult * norm1(mixer(x));  x' = r + mult * norm2(ffn(r))
parallel  (one norm, both sub-layers read its output):
    h = norm1(x);  x' = x + (mixer(h) + ffn(h))
reentry   (no sub-layers; opens a pass over a stretch of layers that runs several times):
    x' = W [x ; x0] + step[turn]         x0: the embedding's rows, turn: the number of the pass
hyper_pre_norm (n copies x_1..x_n of the residual rows instead of one; sub-layer f with coefficients a, b, M):
    u = sum_s a_s x_s;  y = f(c(norm(u)));  x_t' = sum_s M[s, t] x_s + b_t y        c: an optional short
    convolution over time, c(h) = h + conv(h); the model's residual rows are the sum of the copies

The residual stream is float32 for every storage type.  A block leaves the
feed-forward's result as ``pending``: the next norm kernel (of the next block
or the model's final norm) adds it, so every residual sum is one fused pass.
"""
from __future__ import annotations

import dataclasses
from typing import Any, List, Optional

import torch

from .. import ops
from .base import BLOCKS, Delta, FeedForward, Mixer, Part
from .norm import Norm


@dataclasses.dataclass
class ResidualStream:
    x: torch.Tensor                        # [N, width] float32
    act_dtype: torch.dtype
    pending: Optional[Delta] = None        # still to be added to x
    act: Optional[torch.Tensor] = None     # x in the activation dtype, when current
    x0: Optional[torch.Tensor] = None      # the embedding's rows in the activation dtype (models that ask for them)
    turn: int = 0                          # which pass over a stretch of shared layers the running step belongs to
    lanes: Optional[torch.Tensor] = None   # [n, N, width] float32: the copies of a model with several residual streams
    # (mix [n, n], out [n], y [N, width]): the update of the copies that the last sub-layer left to the next reader
    lanes_pending: Optional[tuple] = None

    def settle_lanes(self) -> None:
        """Apply the update of the copies that the last sub-layer left pending."""
        if self.lanes_pending is not None:
            mix, out, y = self.lanes_pending
            ops.hc_write(self.lanes, mix, out, y)
            self.lanes_pending = None

    def fold(self) -> None:
        """A model with several residual streams: x <- their sum (what the final norm and the tools that look at
        the residual rows read); the copies themselves stay as they are."""
        if self.lanes is not None:
            self.settle_lanes()
            ops.hc_sum(self.lanes, out=self.x)
            self.pending, self.act = None, None

    def materialise(self, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x + pending in the activation dtype (all rows, folding pending into x; or only ``rows``)."""
        if rows is None and self.pending is None and self.act is not None:
            return self.act
        n = rows.numel() if rows is not None else self.x.shape[0]
        out = torch.empty((n, self.x.shape[1]), dtype=self.act_dtype, device=self.x.device)
        p = self.pending
        ops.add_norm(self.x, delta=p.value if p else None, delta_bias=p.bias if p else None,
                     parts=p.parts if p else None,
                     resid_out=self.x if (p is not None and rows is None) else None,
                     kind="none", rows=rows, out_act=out)
        if rows is None:
            self.pending, self.act = None, out
        return out


class Block(Part):
    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norm1: Norm, norm2: Norm):
        self.mixer, self.feed_forward, self.norm1, self.norm2 = mixer, feed_forward, norm1, norm2

    def children(self) -> List[Part]:
        return [self.norm1, self.mixer, self.norm2, self.feed_forward]

    def forward(self, stream: ResidualStream, ctx: Any, cache: Any) -> None:
        raise NotImplementedError


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    """r = x + mixer(norm1(x)); x' = r + ffn(norm2(r)).  The feed-forward (and norm2 with it) may be absent."""

    def __init__(self, mixer: Mixer, feed_forward: Optional[FeedForward], norm1: Norm, norm2: Optional[Norm] = None):
        if (feed_forward is None) != (norm2 is None):
            raise ValueError("a block has a second norm exactly when it has a feed-forward")
        super().__init__(mixer, feed_forward, norm1, norm2)

    def children(self) -> List[Part]:
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None]

    def forward(self, stream: ResidualStream, ctx: Any, cache: Any) -> None:
        # A sub-layer that can take its norm and its residual sum into its own kernels does so (steps of a
        # few tokens, where every kernel less shortens the chain); otherwise norm kernel, sub-layer, and the
        # result left pending for the next norm kernel to add.
        x, pending = stream.x, stream.pending
        low = stream.act_dtype != torch.float32
        done = self.mixer.forward_into_residual(x, self.norm1, ctx, cache, pending) if low else False
        if done is False:
            h = self.norm1.apply(x, pending, act_dtype=stream.act_dtype)
            pending = self.mixer.forward(h, ctx, cache)
        else:
            pending = None if done is True else done
        if self.feed_forward is None:
            stream.pending, stream.act = pending, None
            return
        done = self.feed_forward.forward_into_residual(x, self.norm2, ctx, pending) if low else False
        if done is False:
            h = self.norm2.apply(x, pending, act_dtype=stream.act_dtype)
            pending = self.feed_forward.forward(h, ctx)
        else:
            pending = None if done is True else done
        stream.pending = pending
        stream.act = None


@BLOCKS.register("post_norm")
class PostNormBlock(Block):
    def forward(self, stream: ResidualStream, ctx: Any, cache: Any) -> None:
        h = stream.materialise()
        a = self.mixer.forward(h, ctx, cache)
        h = self.norm1.apply(stream.x, a, act_dtype=stream.act_dtype, normalise_residual=True)
        f = self.feed_forward.forward(h, ctx)
        stream.act = self.norm2.apply(stream.x, f, act_dtype=stream.act_dtype, normalise_residual=True)
        stream.pending = None


@BLOCKS.register("norm_after")
class NormAfterBlock(Block):
    """x <- x + mult * norm1(mixer(x)); x <- x + mult * norm2(ffn(x)).  The norms are ``rmsnorm_scalar`` parts (one
    gain each); ``mult`` scales what is added to the residual stream.  The feed-forward may be absent (None).
    The sums and the norms' statistics are float; one kernel per sub-layer normalises its output, adds it to the
    residual rows in place and hands the new rows on in the activation type.  A mixer that declares
    ``reads_residual`` gets the float rows themselves instead of a copy in the activation type."""

    def __init__(self, mixer: Mixer, feed_forward: Optional[FeedForward], norm1: Norm, norm2: Optional[Norm],
                 mult: float = 1.0):
        if (feed_forward is None) != (norm2 is None):
            raise ValueError("a block has a second norm exactly when it has a feed-forward")
        for n in (norm1, norm2):
            if n is not None and not hasattr(n, "gain"):
                raise ValueError("norm_after takes norms with a single gain (rmsnorm_scalar)")
        super().__init__(mixer, feed_forward, norm1, norm2)
        self.mult = float(mult)

    def children(self) -> List[Part]:
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None]

    def forward(self, stream: ResidualStream, ctx: Any, cache: Any) -> None:
        x = stream.x
        if stream.pending is not None:
            stream.materialise()
        if getattr(self.mixer, "reads_residual", False):
            h = x
        else:
            h = stream.materialise()
        a = self.mixer.forward(h, ctx, cache)
        assert a.bias is None and a.parts is None
        act = None
        if self.feed_forward is not None and stream.act_dtype != torch.float32:
            act = torch.empty(x.shape, dtype=stream.act_dtype, device=x.device)
        ops.norm_add(x, a.value, self.norm1.gain, self.mult, self.norm1.eps, ctx.positions, out_act=act)
        stream.act = None
        if self.feed_forward is not None:
            f = self.feed_forward.forward(act if act is not None else x, ctx)
            assert f.bias is None and f.parts is None
            ops.norm_add(x, f.value, self.norm2.gain, self.mult, self.norm2.eps, ctx.positions)
        stream.pending = None


@BLOCKS.register("parallel")
class ParallelBlock(Block):
    """h = norm1(x); x <- x + (mixer(h) + ffn(h)): one norm, and both sub-layers read its output.  The feed-forward
    may be absent.  The mixer's result (activation type) and the feed-forward's (float, when it can leave it so) are
    left pending together: the next norm kernel forms their sum and adds it to the float residual rows."""

    def __init__(self, mixer: Mixer, feed_forward: Optional[FeedForward], norm1: Norm):
        super().__init__(mixer, feed_forward, norm1, None)

    def children(self) -> List[Part]:
        return [p for p in (self.norm1, self.mixer, self.feed_forward) if p is not None]

    def forward(self, stream: ResidualStream, ctx: Any, cache: Any) -> None:
        h = self.norm1.apply(stream.x, stream.pending, act_dtype=stream.act_dtype)
        a = self.mixer.forward(h, ctx, cache)
        assert a.bias is None and a.parts is None
        pending = a
        if self.feed_forward is not None:
            f = self.feed_forward.forward(h, ctx)
            assert f.bias is None
            if f.parts is not None:
                assert f.value is None
                pending = Delta(a.value, None, f.parts)
            elif f.value.dtype == torch.float32 and f.value.is_contiguous():
                pending = Delta(a.value, None, f.value.unsqueeze(0))
            else:
                # the feed-forward's result in the activation type: one more pass adds the mixer's to the residual
                # rows first (the two are not summed in the activation type)
                ops.add_norm(stream.x, delta=a.value, resid_out=stream.x, kind="none", act_dtype=stream.act_dtype)
                pending = f
        stream.pending, stream.act = pending, None


@BLOCKS.register("reentry")
class ReentryBlock(Block):
    """Opens a pass over a stretch of layers that runs several times with the same weights:
    x <- W [x ; x0] + step[turn], with x0 the embedding's rows (``ResidualStream.x0``), W [width, 2 * width] (x's
    columns first) and step [passes, width]; ``ResidualStream.turn`` says which pass begins.  The product's float
    result becomes the residual stream; the step vector is left pending for the next norm kernel.  It has no mixer,
    no cache and no norm."""

    wants_embedding = True

    def __init__(self, width: int, passes: int, in_name: str, step_name: str):
        super().__init__(None, None, None, None)
        self.width, self.passes, self.in_name, self.step_name = width, passes, in_name, step_name
        self.w_in = self.step = None

    def children(self) -> List[Part]:
        return []

    def param_specs(self):
        from ..weights.spec import MATRIX, VECTOR, ParamSpec
        return [ParamSpec(self.in_name, (self.width, 2 * self.width), MATRIX),
                ParamSpec(self.step_name, (self.passes, self.width), VECTOR)]

    def bind(self, tensors) -> None:
        self.w_in, self.step = tensors[self.in_name], tensors[self.step_name]

    def param_bytes(self) -> int:
        return self.w_in.numel() * self.w_in.element_size() + 4 * self.width

    def forward(self, stream: ResidualStream, ctx: Any, cache: Any) -> None:
        if stream.x0 is None:
            raise RuntimeError("a reentry block needs the embedding's rows (ResidualStream.x0)")
        both = ops.concat_rows(stream.materialise(), stream.x0)
        stream.x = ops.linear(both, self.w_in, out_dtype=torch.float32)
        stream.pending, stream.act = Delta(None, self.step[stream.turn]), None


@BLOCKS.register("hyper_pre_norm")
class HyperPreNormBlock(Block):
    """A pre-norm block over ``streams`` copies of the residual rows ("hyper-connections").  For each of its two
    sub-layers (the mixer, then the feed-forward, which may be absent) with the tensors ``<hc>.in`` [n], ``<hc>.out``
    [n] and ``<hc>.mix`` [n, n] (indexed [from, to]):

        u = sum_s in[s] x_s;   h = norm(u);   h <- h + conv(h) (``canon_names``: a filter [width, taps] per
        sub-layer, or None);   y = sub-layer(h);   x_t <- sum_s mix[s, t] x_s + out[t] y   for all t at once.  The update is left pending
        (``ResidualStream.lanes_pending``) and done by the kernel that reads the copies next, in the same pass.

    The copies start as the embedding's rows (made by the first block that runs) and ``ResidualStream.fold`` sums
    them.  Mixture, norm statistics, the convolution and the update are float arithmetic on float rows; the
    sub-layers get h in the activation type.  Per request the block keeps the convolutions' last taps - 1 inputs in
    state slots of its own beside the mixer's cache: its cache entry is (state 1, the mixer's need, state 2)."""

    def __init__(self, mixer: Mixer, feed_forward: Optional[FeedForward], norm1: Norm, norm2: Optional[Norm],
                 streams: int, width: int, hc_names: tuple, canon_names: Optional[tuple] = None, taps: int = 1):
        if (feed_forward is None) != (norm2 is None):
            raise ValueError("a block has a second norm exactly when it has a feed-forward")
        if streams < 1:
            raise ValueError("a model has at least one residual stream")
        if canon_names is not None and taps < 1:
            raise ValueError("a convolution needs at least one tap")
        super().__init__(mixer, feed_forward, norm1, norm2)
        self.streams, self.width, self.taps = int(streams), int(width), int(taps)
        self.hc_names, self.canon_names = tuple(hc_names), (tuple(canon_names) if canon_names else None)
        self.n_sub = 1 if feed_forward is None else 2
        self.coef = [None, None]
        self.filters = [None, None]

    def children(self) -> List[Part]:
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None]

    def param_specs(self):
        from ..weights.spec import VECTOR, ParamSpec
        n, specs = self.streams, []
        for i in range(self.n_sub):
            hc = self.hc_names[i]
            specs += [ParamSpec(hc + ".in", (n,), VECTOR), ParamSpec(hc + ".out", (n,), VECTOR),
                      ParamSpec(hc + ".mix", (n, n), VECTOR)]
            if self.canon_names is not None:
                specs.append(ParamSpec(self.canon_names[i], (self.width, self.taps), VECTOR))
        return specs

    def bind(self, tensors) -> None:
        for i in range(self.n_sub):
            hc = self.hc_names[i]
            self.coef[i] = tuple(tensors[hc + k].to(torch.float32).contiguous() for k in (".in", ".mix", ".out"))
            if self.canon_names is not None:
                self.filters[i] = tensors[self.canon_names[i]].to(torch.float32).contiguous()

    def param_bytes(self) -> int:
        return 4 * self.n_sub * (self.width * self.taps if self.canon_names is not None else 0)

    def cache_spec(self):
        from .base import StateSpec
        tail = StateSpec((self.taps - 1, self.width), torch.float32) \
            if self.canon_names is not None and self.taps > 1 else None
        return (tail, self.mixer.cache_spec(), tail if self.n_sub == 2 else None)

    def _input(self, i: int, stream: ResidualStream, norm: Norm, ctx: Any, tail: Any) -> torch.Tensor:
        a, _, _ = self.coef[i]
        if self.canon_names is not None and tail is not None and getattr(ctx, "single_tokens", False):
            # every request brings one token: pending update, read, norm and convolution in one kernel
            out = torch.empty(stream.x.shape, dtype=stream.act_dtype, device=stream.x.device)
            pending, stream.lanes_pending = stream.lanes_pending, None
            return ops.hc_step_conv(stream.lanes, pending, a, norm.gamma, norm.eps, self.filters[i], tail.state, out,
                                    ctx.positions, ctx.seq_of_token, ctx.slots, write_state=tail.writable)
        if stream.lanes_pending is not None:
            # the update the sub-layer before left pending and this read in one pass over the copies
            mix, out_coef, y = stream.lanes_pending
            stream.lanes_pending = None
            h = ops.hc_write_read_norm(stream.lanes, mix, out_coef, y, a, norm.gamma, norm.eps, ctx.positions)
        else:
            h = ops.hc_read_norm(stream.lanes, a, norm.gamma, norm.eps, ctx.positions)
        out = torch.empty(h.shape, dtype=stream.act_dtype, device=h.device)
        if self.canon_names is None:
            if stream.act_dtype == torch.float32:
                return h
            ops.add_norm(h, kind="none", out_act=out)
            return out
        state = tail.state if tail is not None else h.new_zeros((1, 0, self.width))
        ops.conv_residual(h, self.filters[i], state, out, ctx.positions, ctx.seq_of_token, ctx.q_start, ctx.slots)
        return out

    @staticmethod
    def _rows(delta: Delta, stream: ResidualStream) -> torch.Tensor:
        """What a sub-layer left, as one tensor of rows (float or the activation type)."""
        if delta.bias is None and delta.parts is None:
            return delta.value
        if delta.bias is None and delta.value is None and delta.parts.shape[0] == 1:
            return delta.parts[0]
        y = torch.zeros(stream.x.shape, dtype=torch.float32, device=stream.x.device)
        ops.add_norm(y, delta=delta.value, delta_bias=delta.bias, parts=delta.parts, resid_out=y, kind="none",
                     act_dtype=stream.act_dtype)
        return y

    def forward(self, stream: ResidualStream, ctx: Any, cache: Any) -> None:
        if stream.lanes is None:
            if stream.pending is not None:
                stream.materialise()
            stream.lanes = ops.hc_spread(stream.x, self.streams)
        tail1, mixer_cache, tail2 = cache
        h = self._input(0, stream, self.norm1, ctx, tail1)
        y = self._rows(self.mixer.forward(h, ctx, mixer_cache), stream)
        # the update of the copies is left to the next reader (the next sub-layer's read, or ``fold``)
        stream.lanes_pending = (self.coef[0][1], self.coef[0][2], y)
        if self.feed_forward is not None:
            h = self._input(1, stream, self.norm2, ctx, tail2)
            y = self._rows(self.feed_forward.forward(h, ctx), stream)
            stream.lanes_pending = (self.coef[1][1], self.coef[1][2], y)
        stream.pending, stream.act = None, None
