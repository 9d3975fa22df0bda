"""Arrangements of a layer's parts around the residual stream.

`pre_norm` is GPT-2's: `x -> norm1 -> mixer -> +x -> norm2 -> feed-forward -> +x`, the residual
sums in float32 (graph_ir.cpp:732-756, the sequential branch; operand order x then the
branch's output, :754-756).  The mixer and the feed-forward add into the stream themselves so that
their last projection can do the sum in its epilogue.  A layer of this arrangement may have no
feed-forward (and then no second norm), and may add further things to the stream after its sublayers
(`LayerSpec.addons`).

`sandwich` norms every sublayer on both sides: `x -> x + after_mixer(mixer(norm1(x)))`, then
`x -> x + after_ffn(ffn(norm2(x)))`.  A sublayer's output cannot be added by its last projection
here (it is normed first), so the sublayer hands over its output as a weighted sum of float32
rows (`branches`) and the norm after it sums, norms and adds in one launch.  A layer of this
arrangement may have no feed-forward; it then has no norms around one either.

`shared_norm` has one norm that both sublayers read: `h = norm1(x)`, `x -> x + mixer(h) + ffn(h)`.
The mixer's last projection adds into the stream and the feed-forward's adds into that, both in
float32; a layer of this arrangement may have no feed-forward.
"""
from __future__ import annotations

from .base import Block, register_part


class PreNormBlock(Block):
    def __init__(self, norm1, mixer, norm2, ffn, **more_norms):
        if norm1 is None or more_norms or (ffn is None) != (norm2 is None):
            raise ValueError("block 'pre_norm' has a norm before the mixer and, with a feed-forward, one before that")
        super().__init__(norm1, mixer, norm2, ffn)


    def forward(self, ctx, x, app):
        announce = getattr(ctx.ops, "announce_weights", None)
        if announce is not None:    # a hint: this block's matrices in the order they are streamed, then what follows
            announce(self.mixer.stream_weights() + (self.ffn.stream_weights() if self.ffn is not None else [])
                     + list(getattr(ctx, "next_weights", ())))
        h = self.norm1.forward(ctx, x, ctx.dtype)
        x = self.mixer.forward(ctx, h, x, app)
        if self.ffn is not None:
            h = self.norm2.forward(ctx, x, ctx.dtype)
            x = self.ffn.forward(ctx, h, x)
        return self.add_ons(ctx, x)


class SandwichBlock(Block):
    def __init__(self, norm1, mixer, norm2, ffn, after_mixer=None, after_ffn=None, **more_norms):
        if norm1 is None or after_mixer is None or more_norms:
            raise ValueError("block 'sandwich' has a norm before the mixer and one named 'after_mixer'")
        if (ffn is None) != (norm2 is None) or (ffn is None) != (after_ffn is None):
            raise ValueError("block 'sandwich' has a feed-forward with a norm before it and one named 'after_ffn', "
                             "or none of the three")
        extra = {"after_mixer": after_mixer} if ffn is None else {"after_mixer": after_mixer, "after_ffn": after_ffn}
        super().__init__(norm1, mixer, norm2, ffn, **extra)

    def forward(self, ctx, x, app):
        announce = getattr(ctx.ops, "announce_weights", None)
        if announce is not None:
            announce(self.mixer.stream_weights() + (self.ffn.stream_weights() if self.ffn is not None else [])
                     + list(getattr(ctx, "next_weights", ())))
        h = self.norm1.forward(ctx, x, ctx.dtype)
        x = self.more_norms["after_mixer"].add_normed(ctx, x, self.mixer.branches(ctx, h, app))
        if self.ffn is None:
            return x
        h = self.norm2.forward(ctx, x, ctx.dtype)
        return self.more_norms["after_ffn"].add_normed(ctx, x, self.ffn.branches(ctx, h))


class SharedNormBlock(Block):
    def __init__(self, norm1, mixer, norm2, ffn, **more_norms):
        if norm1 is None or norm2 is not None or more_norms:
            raise ValueError("block 'shared_norm' has exactly one norm, which the mixer and the feed-forward both read")
        super().__init__(norm1, mixer, None, ffn)

    def forward(self, ctx, x, app):
        announce = getattr(ctx.ops, "announce_weights", None)
        if announce is not None:
            announce(self.mixer.stream_weights() + (self.ffn.stream_weights() if self.ffn is not None else [])
                     + list(getattr(ctx, "next_weights", ())))
        h = self.norm1.forward(ctx, x, ctx.dtype)
        x = self.mixer.forward(ctx, h, x, app)
        return x if self.ffn is None else self.ffn.forward(ctx, h, x)


register_part("block", "pre_norm", PreNormBlock)
register_part("block", "shared_norm", SharedNormBlock)
register_part("block", "sandwich", SandwichBlock)
