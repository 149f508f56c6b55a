"""A layer arrangement with several residual streams ("hyper-connections").

Instead of one stream x the model keeps S streams x_1 .. x_S, all equal to the embedding's output at the
start.  Each sublayer q (the mixer, then the feed-forward) has three small weights: `in` [S], `out` [S] and
`mix` [S, S] (indexed [from, to]).  It reads u = sum_s in[s] x_s, computes y = sublayer(norm(u)), and then all
streams change at once from the old ones: x_t <- sum_s mix[s, t] x_s + out[t] y.  After the last layer the
stream is the sum of the S streams.  With S = 1, in = out = mix = 1 this is the ordinary pre-norm layer.

One kernel runs between two sublayers (`ops.hc_step`): it applies the update that the finished sublayer left,
reads the next sublayer's u out of the new streams and norms it.  The update of a layer's last sublayer is
therefore left pending (in `ctx.extra`) for the block of the next layer, or for `finish`, which applies it
and returns the sum.  Streams, sums and norm statistics are fp32.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Block, WeightDecl, register_block
from .norm import RMSNorm

_KEY = "hyper_streams"


@register_block("hyper_connections")
class HyperConnectionsBlock(Block):
    def __init__(self, streams: int, has_ffn: bool = True):
        self.S, self.has_ffn = int(streams), bool(has_ffn)
        if not 1 <= self.S <= 8:
            raise ValueError(f"hyper_connections: {self.S} streams; the kernel takes 1 to 8")

    def weight_decls(self):
        S = self.S
        decls = {}
        for q in (("1", "2") if self.has_ffn else ("1",)):
            decls["in" + q] = WeightDecl((S,), role="vector", init="norm")
            decls["out" + q] = WeightDecl((S,), role="vector", init="norm")
            decls["mix" + q] = WeightDecl((S, S), role="vector")
        return decls

    # ---- the state between layers: the streams, the buffer sublayers add into, and the pending update ------------
    def _state(self, ctx, x):
        st = ctx.extra.get(_KEY)
        if st is None or st["x"] is not x:
            T, d = x.shape
            st = ctx.extra[_KEY] = dict(x=x, X=torch.empty((self.S, T, d), dtype=torch.float32, device=x.device),
                                        y=torch.zeros((T, d), dtype=torch.float32, device=x.device), fresh=True, pending=None)
        return st

    def _read(self, ctx, st, in_w, norm):
        """Applies what is pending and returns the normed input of the sublayer that reads with `in_w`."""
        X, y = st["X"], st["y"]
        h = torch.empty(y.shape, dtype=ctx.act_dtype, device=y.device)
        fused = isinstance(norm, RMSNorm)
        u = None if fused else torch.empty_like(y)
        kw = dict(in_w=in_w, h_out=h if fused else None, u_out=u, norm_w=norm.w["weight"] if fused else None,
                  eps=norm.eps if fused else 0.0)
        if st["fresh"]:
            ops.hc_step(X, x_init=st["x"], **kw)
            st["fresh"] = False
        elif st["pending"] is not None:
            mix, out_w = st["pending"]
            ops.hc_step(X, y=y, mix=mix, out_w=out_w, **kw)
            st["pending"] = None
        else:
            ops.hc_step(X, **kw)
        return h if fused else norm.forward(ctx, u)

    def forward(self, ctx, x, layer, cache, reads_only=False, next_norm=None):
        st = self._state(ctx, x)
        w = self.w
        h = self._read(ctx, st, w["in1"], layer.mixer_norm)
        layer.mixer.forward(ctx, cache, h, st["y"], reads_only)
        st["pending"] = (w["mix1"], w["out1"])
        if layer.ffn is not None:
            h = self._read(ctx, st, w["in2"], layer.ffn_norm)
            layer.ffn.forward(ctx, h, st["y"])
            st["pending"] = (w["mix2"], w["out2"])

    def finish(self, ctx, x):
        st = ctx.extra.get(_KEY)
        if st is None or st["x"] is not x:
            return x
        X, y = st["X"], st["y"]
        u = torch.empty_like(y)
        if st["fresh"]:
            ops.hc_step(X, x_init=x, u_out=u)
            st["fresh"] = False
        elif st["pending"] is not None:
            mix, out_w = st["pending"]
            ops.hc_step(X, y=y, mix=mix, out_w=out_w, u_out=u)
            st["pending"] = None
        else:
            ops.hc_step(X, u_out=u)
        return u
