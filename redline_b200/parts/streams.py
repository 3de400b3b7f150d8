"""Several residual streams (hyper-connections) and the block that runs its sublayers on them.

Instead of one stream a token has ``streams`` of them, X_1 .. X_n, all equal to the embedding at the start.
A sublayer has a connection (three small tensors): it reads u = sum_s in[s] X_s, runs y = f(norm(u)), and
writes back X_t <- sum_s mix[s, t] X_s + out[t] y for all t at once from the old streams.  After the last
layer the model's stream is the sum of the X_s.  With one stream, in = out = mix = 1, this is the pre-norm
residual block.

The streams [tokens, n, width] live in float32 in the workspace.  One kernel per sublayer boundary
(csrc/stream_ops.cu) writes a sublayer's output back and forms the next sublayer's normed input, across
blocks too (``ctx.block_normed``); the last block's last kernel also writes the streams' sum into the
model's residual buffer, which the final norm reads.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict

import torch

from ..ops import kernels
from .base import Block, Part, op_mark, register
from .spec import TensorSpec


@dataclass(frozen=True)
class StreamConnectionParams:
    streams: int


@register("connection", "stream_connection")
class StreamConnection(Part):
    """How one sublayer reads the streams (``in`` [n]) and writes them back (``mix`` [n, n] indexed
    (from, to), ``out`` [n]); kept in float32."""

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        if not 1 <= self.params.streams <= kernels.MAX_STREAMS:
            raise ValueError(f"between 1 and {kernels.MAX_STREAMS} residual streams; got {self.params.streams}")

    def tensors(self) -> Dict[str, TensorSpec]:
        n = self.params.streams
        return {"in": TensorSpec((n,)), "out": TensorSpec((n,)), "mix": TensorSpec((n, n))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.read_in = tensors["in"].float().contiguous()
        self.out = tensors["out"].float().contiguous()
        self.mix = tensors["mix"].float().contiguous()

    def nbytes(self) -> int:
        return 4 * (self.read_in.numel() + self.out.numel() + self.mix.numel())


@register("block", "hyper")
class HyperBlock(Block):
    """Pre-norm sublayers on several residual streams.  ``mixer_conn`` / ``ffn_conn`` are set by the model
    builder from the layer's spec; the norms must be RMS norms (the boundary kernel applies them)."""

    keeps_streams = True

    def first_norm(self):
        return self.mixer_norm

    def _streams(self, residual, ctx) -> torch.Tensor:
        rt = self.rt
        n = self.mixer_conn.params.streams
        return rt.workspace.get("hyper.streams", (rt.max_tokens, n, residual.shape[1]), torch.float32)[:ctx.T]

    def _boundary(self, ctx, streams, x, *, init=None, y=None, conn=None, nxt=None, total=None) -> None:
        """Writes sublayer output ``y`` back through ``conn`` and forms the input of the sublayer ``nxt`` =
        (its connection, its norm) in ``x``."""
        read_in = norm_w = None
        eps = 0.0
        if nxt is not None:
            read_in = nxt[0].read_in
            norm_w, eps = nxt[1].rms_params()
        kernels.streams_step(streams, ctx.T, init=init, y=y, mix=conn.mix if conn is not None else None,
                             out_w=conn.out if conn is not None else None, read_in=read_in, norm_w=norm_w, eps=eps,
                             normed=x if nxt is not None else None, total=total)
        n, w = streams.shape[1], streams.shape[2]
        moved = (n * w * 4.0) * ((1 if init is None else 0) + (1 if (y is not None or init is not None) else 0))
        moved += w * ((x.element_size() if nxt is not None else 0) + (y.element_size() if y is not None else 0)
                      + (4 if total is not None else 0) + (4 if init is not None else 0))
        op_mark(ctx, "streams_mix+rmsnorm", nbytes=ctx.T * moved)

    def forward(self, residual, pending, ctx, cache, state):
        if pending is not None:
            raise ValueError("a block with several streams takes nothing pending from the block before it")
        for norm in (self.mixer_norm, self.ffn_norm):
            if norm is not None and norm.rms_params() is None:
                raise ValueError("the hyper block's norms are RMS norms")
        rt = self.rt
        T = ctx.T
        ctx.block_hand = None
        ready, ctx.block_normed = ctx.block_normed, None
        streams = self._streams(residual, ctx)
        x = rt.workspace.get("block.normed", (rt.max_tokens, residual.shape[1]), rt.dtype)[:T]
        if not (ready is not None and ready[0] is self.mixer_norm):
            # the model's first block, or one behind a block that keeps one stream: every stream starts as a copy
            self._boundary(ctx, streams, x, init=residual, nxt=(self.mixer_conn, self.mixer_norm))
        a = self.mixer.forward(x, ctx, cache, state)
        # what comes after this block: another block of this kind takes its first input from this block's last kernel
        nb = ctx.block_next
        after = (nb.mixer_conn, nb.mixer_norm) if isinstance(nb, HyperBlock) and \
            nb.mixer_conn.params.streams == self.mixer_conn.params.streams else None
        last = residual if after is None else None          # the streams' sum, for whoever reads one stream next
        if self.ffn is None:
            self._boundary(ctx, streams, x, y=a, conn=self.mixer_conn, nxt=after, total=last)
        else:
            self._boundary(ctx, streams, x, y=a, conn=self.mixer_conn, nxt=(self.ffn_conn, self.ffn_norm))
            f = self.ffn.forward(x, ctx)
            self._boundary(ctx, streams, x, y=f, conn=self.ffn_conn, nxt=after, total=last)
        if after is not None:
            ctx.block_normed = (nb.mixer_norm, x)
        return None
