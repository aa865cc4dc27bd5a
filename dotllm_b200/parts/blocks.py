"""Block arrangements: how a layer's parts meet the residual stream.

"pre_norm" is the reference's wiring, r=h; h=r+mixer(norm(h)); r=h; h=r+ffn(norm(h))
(src/DotLLM.Models/Architectures/TransformerModel.cs:185-392).  As in the reference's GPU path
(src/DotLLM.Cuda/CudaTransformerModel.cs:252-286) each residual add is folded into the norm
that follows it, across the layer boundary too: a block returns its last branch output still
to be added ("pending"), and whoever normalises next adds it.
"""
from __future__ import annotations

from .base import Arrangement, normalised_for, register_arrangement


class PreNormBlock(Arrangement):
    """The feed-forward and its norm may be absent (a layer that only mixes): the mixer's branch is handed on."""
    needs = ("mixer_norm", "mixer")
    narrows = True

    def forward(self, residual, pending, step, cache_view, keep_rows=None):
        n = normalised_for(self.mixer, self.mixer_norm, residual, pending)
        a = self.mixer.forward(n, step, cache_view)          # every token: the cache needs all keys and values
        if keep_rows is not None:
            # nothing after this layer reads the other rows: the output projection, the second norm and
            # the feed-forward run on the kept rows only
            from ..kernels import ops
            residual = ops.gather_rows(residual, keep_rows)
            a = ops.narrow_rows(a, keep_rows)
        if "feed_forward" not in self.parts:
            return residual, a
        n = normalised_for(self.feed_forward, self.feed_forward_norm, residual, a)
        return residual, self.feed_forward.forward(n)


class SandwichNormBlock(Arrangement):
    """A norm before and behind each sublayer: h += post(mixer(pre(h))); h += post(ff(pre(h))).  The
    feed-forward and its two norms may be absent (a layer that only mixes).  A sublayer's output is handed
    on with its post-norm still to be applied (``Norm.branch``): the norm that reads the stream next
    normalises the branch, adds it and normalises the sum in one kernel, across the layer boundary too."""
    needs = ("mixer_norm", "mixer", "mixer_post_norm")
    narrows = True

    def forward(self, residual, pending, step, cache_view, keep_rows=None):
        n = normalised_for(self.mixer, self.mixer_norm, residual, pending)
        branch = self.mixer_post_norm.branch(self.mixer.forward(n, step, cache_view))
        if keep_rows is not None:
            from ..kernels import ops
            residual = ops.gather_rows(residual, keep_rows)
            branch = ops.narrow_rows(branch, keep_rows)
        if "feed_forward" not in self.parts:
            return residual, branch
        n = normalised_for(self.feed_forward, self.feed_forward_norm, residual, branch)
        return residual, self.feed_forward_post_norm.branch(self.feed_forward.forward(n))


class ParallelBlock(Arrangement):
    """One norm, two sublayers that both read its output, one addition: h = norm(x); x += mixer(h) + ff(h).  The
    feed-forward may be absent.  The mixer's output joins the stream at once (its last product adds itself where it
    can); the feed-forward's is handed on as the pending branch, so the stream gets x + mixer + ff in float32."""
    needs = ("norm", "mixer")
    narrows = True

    def forward(self, residual, pending, step, cache_view, keep_rows=None):
        from ..kernels import ops
        n = ops.resolve(normalised_for(None, self.norm, residual, pending))     # a plain tensor: two parts read it
        a = self.mixer.forward(n, step, cache_view)         # every token: the cache needs all keys, values and states
        if keep_rows is not None:
            residual = ops.gather_rows(residual, keep_rows)
            a = ops.narrow_rows(a, keep_rows)
            if "feed_forward" in self.parts:
                n = ops.gather_rows(n, keep_rows, out_dtype=n.dtype)
        if "feed_forward" not in self.parts:
            return residual, a
        if not (isinstance(a, ops.PendingProduct) and a.add_into(residual)):
            ops.add_rows(residual, ops.resolve(a).to(residual.dtype))
        return residual, self.feed_forward.forward(n)


class ConnectedBlock(Arrangement):
    """Pre-norm sublayers that meet the stream through connections of their own (``parts.connections``): what a
    sublayer's norm reads and how its output joins are the connection's business, so the stream may be several copies
    with read, write and mixing weights per sublayer, or one stream with a gain on every branch.  A sublayer's output is
    handed on unadded; the next read (the next layer's, or the model's last norm) adds it.  The feed-forward with its norm
    and connection may be absent."""
    needs = ("mixer_norm", "mixer", "mixer_connection")
    narrows = True

    def forward(self, residual, pending, step, cache_view, keep_rows=None):
        n = self.mixer_connection.read(self.mixer_norm, residual, pending)
        branch = self.mixer_connection.write(self.mixer.forward(n, step, cache_view))   # every token: the cache needs them all
        if keep_rows is not None:
            from ..kernels import ops
            residual = ops.gather_rows(residual, keep_rows)
            branch = ops.narrow_rows(branch, keep_rows)
        if "feed_forward" not in self.parts:
            return residual, branch
        n = self.feed_forward_connection.read(self.feed_forward_norm, residual, branch)
        return residual, self.feed_forward_connection.write(self.feed_forward.forward(n))


register_arrangement("pre_norm", PreNormBlock)
register_arrangement("connected", ConnectedBlock)
register_arrangement("parallel", ParallelBlock)
register_arrangement("sandwich_norm", SandwichNormBlock)
