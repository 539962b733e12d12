"""The arrangements of a layer.

`pre_norm`: x += mixer(norm(x)); x += feed_forward(norm(x))  (src/model/decoder_layer.cpp:63-98).
The hidden state travels as (residual, delta): each sum is done by the next norm's
kernel, which writes the new residual and its normalised copy in one pass.

`sandwich_norm`: a norm before and a norm after every sublayer, x += norm_b(mixer(norm_a(x))),
then the same around the feed-forward (which a layer may lack), on a hidden state that is kept
in float32 whatever the compute type.  Here `delta` is a `NormedBranch`: a sublayer's output
that still has to be normalised and added.  Whoever comes next does it (the next block, a
stream step or the model's tail), in the same kernel that normalises the sum for its own
input, so a layer costs two passes over the hidden state.
"""
from __future__ import annotations

from ..config.plan import PartSpec
from .base import Part, build_part, register_part


class PreNormBlock(Part):
    def __init__(self, mixer, feed_forward, norm: PartSpec, mixer_norm_name: str, feed_forward_norm_name: str):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm = build_part("norm", norm)
        self.feed_forward_norm = build_part("norm", norm)
        self.mixer_norm_name, self.feed_forward_norm_name = mixer_norm_name, feed_forward_norm_name

    def weight_specs(self, prefix: str) -> dict:
        specs = {}
        specs.update(self.mixer_norm.weight_specs(prefix + self.mixer_norm_name))
        specs.update(self.feed_forward_norm.weight_specs(prefix + self.feed_forward_norm_name))
        specs.update(self.mixer.weight_specs(prefix))
        specs.update(self.feed_forward.weight_specs(prefix))
        return specs

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        self.mixer_norm.bind(weights, prefix + self.mixer_norm_name, dtype, device)
        self.feed_forward_norm.bind(weights, prefix + self.feed_forward_norm_name, dtype, device)
        self.mixer.bind(weights, prefix, dtype, device)
        self.feed_forward.bind(weights, prefix, dtype, device)

    def forward(self, residual, delta, ctx, cache):
        normed = ctx.scratch.get("block.normed", residual.shape, ctx.dtype)
        self.mixer_norm(residual, normed, delta)
        mixed = self.mixer.forward(normed, ctx, cache)
        self.feed_forward_norm(residual, normed, mixed)
        return residual, self.feed_forward.forward(normed, ctx)


class NormedBranch:
    """A sublayer's output (compute type) that is still to be normalised with `norm` and added to the float32 stream."""

    def __init__(self, branch, norm):
        self.branch, self.norm = branch, norm


def settle(residual, pending, norm=None, out=None):
    """stream += norm_b(branch) for a pending `NormedBranch` (None: nothing to add), and, with `norm` and `out`,
    out = norm(stream) of the sum: one kernel."""
    from ..csrc import ops
    if pending is not None and not isinstance(pending, NormedBranch):
        raise TypeError("a float32 stream takes a NormedBranch as its pending sum")
    if pending is None and norm is None:
        return out
    return ops.sandwich_norm(residual, pending.branch if pending else None, pending.norm.weight if pending else None,
                             pending.norm.eps if pending else 0.0, norm.weight if norm else None,
                             norm.eps if norm else 0.0, out)


class SandwichNormBlock(Part):
    stream_dtype = "float32"

    def __init__(self, mixer, feed_forward, norm: PartSpec, names=("norm1", "norm1b", "norm2", "norm2b")):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.names = tuple(names)
        self.norms = [build_part("norm", norm) for _ in range(4 if feed_forward is not None else 2)]

    def weight_specs(self, prefix: str) -> dict:
        specs = {}
        for part, name in zip(self.norms, self.names):
            specs.update(part.weight_specs(prefix + name))
        specs.update(self.mixer.weight_specs(prefix))
        if self.feed_forward is not None:
            specs.update(self.feed_forward.weight_specs(prefix))
        return specs

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        for part, name in zip(self.norms, self.names):
            part.bind(weights, prefix + name, dtype, device)
        self.mixer.bind(weights, prefix, dtype, device)
        if self.feed_forward is not None:
            self.feed_forward.bind(weights, prefix, dtype, device)

    def forward(self, residual, delta, ctx, cache):
        normed = ctx.scratch.get("block.normed", residual.shape, ctx.dtype)
        settle(residual, delta, self.norms[0], normed)
        pending = NormedBranch(self.mixer.forward(normed, ctx, cache), self.norms[1])
        if self.feed_forward is None:
            return residual, pending
        settle(residual, pending, self.norms[2], normed)
        return residual, NormedBranch(self.feed_forward.forward(normed, ctx), self.norms[3])


class ShiftSandwichBlock(Part):
    """Sandwich-norm sublayers on a float32 stream, x += norm_b(mixer(shift(norm_a(x)))), then the same around the
    feed-forward without the shift (a layer may lack it), with norms of any kind that `ops.settle_norm` takes.

    Token shift: what the mixer reads, h, becomes h_t + (h_(t-1) - h_t) * mu with mu the vector `shift_name`, h_(t-1) the
    row before it in the sequence as it was before this step (zeros before the first token).  The last h of a sequence
    is part of its state: `state_size` float32 values per sequence in the layer's cache (`LayerCache.block_state`).

    Token side input (`side`, optional), after the feed-forward: with e the columns [index * dim, (index + 1) * dim) of
    a second embedding table that all layers share, g = gelu_tanh(W_gate x) * e, y = W_proj g and
    x += y / sqrt(mean(y^2) + eps) * w.  `side` = {table, vocab, columns, dim, index, eps, gate, proj, norm}, the names
    relative to the layer's prefix but for `table`.

    Every sum is left pending and done by the next reader's kernel, which normalises the sum for its own input."""
    stream_dtype = "float32"

    def __init__(self, mixer, feed_forward, norm: PartSpec, hidden_size: int, names=("norm1", "norm1b", "norm2", "norm2b"),
                 shift_name: str = "shift", side=None):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.hidden_size, self.names, self.shift_name = int(hidden_size), tuple(names), shift_name
        self.norms = [build_part("norm", norm) for _ in range(4 if feed_forward is not None else 2)]
        self.state_size = self.hidden_size
        self.mu = None
        self.side = dict(side) if side else None
        self.side_norm = self.side_table = self.w_side_gate = self.w_side_proj = None
        if self.side:
            self.side_norm = build_part("norm", PartSpec("rms_norm", {"size": self.hidden_size, "eps": self.side["eps"]}))

    def weight_specs(self, prefix: str) -> dict:
        from ..weights.loader import WeightSpec
        specs, H = {}, self.hidden_size
        for part, name in zip(self.norms, self.names):
            specs.update(part.weight_specs(prefix + name))
        specs[prefix + self.shift_name] = WeightSpec((H,), "bias")
        if self.side:
            sd = self.side
            specs[sd["table"]] = WeightSpec((sd["vocab"], sd["columns"]))
            specs[prefix + sd["gate"]] = WeightSpec((sd["dim"], H))
            specs[prefix + sd["proj"]] = WeightSpec((H, sd["dim"]))
            specs.update(self.side_norm.weight_specs(prefix + sd["norm"]))
        specs.update(self.mixer.weight_specs(prefix))
        if self.feed_forward is not None:
            specs.update(self.feed_forward.weight_specs(prefix))
        return specs

    def ignorable(self, prefix: str):
        """The norms of a feed-forward that the layer does not have may be stored all the same."""
        if self.feed_forward is not None:
            return []
        return [n for name in self.names[2:] for n in self.norms[0].weight_specs(prefix + name)]

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        import torch
        for part, name in zip(self.norms, self.names):
            part.bind(weights, prefix + name, dtype, device)
        self.mu = weights[prefix + self.shift_name].to(device=device, dtype=torch.float32).contiguous()
        if self.side:
            sd = self.side
            self.side_table = weights[sd["table"]]           # one tensor for all layers: not taken out of `weights`
            self.w_side_gate = weights.pop(prefix + sd["gate"]).contiguous()
            self.w_side_proj = weights.pop(prefix + sd["proj"]).contiguous()
            self.side_norm.bind(weights, prefix + sd["norm"], dtype, device)
        self.mixer.bind(weights, prefix, dtype, device)
        if self.feed_forward is not None:
            self.feed_forward.bind(weights, prefix, dtype, device)

    @staticmethod
    def _settle(residual, pending, norm, out):
        from ..csrc import ops
        if pending is not None and not isinstance(pending, NormedBranch):
            raise TypeError("a float32 stream takes a NormedBranch as its pending sum")
        return ops.settle_norm(residual, pending.branch if pending else None, pending.norm if pending else None, norm, out)

    def forward(self, residual, delta, ctx, cache):
        import torch
        from ..csrc import ops
        from .linear import linear
        N, H = ctx.n_tokens, self.hidden_size
        if cache.block_state is None:
            raise ops.KernelError("the token shift keeps a row per sequence: the cache was built without block_state")
        h = ctx.scratch.get("block.h32", (N, H), torch.float32)
        self._settle(residual, delta, self.norms[0], h)
        shifted = ctx.scratch.get("block.normed", (N, H), ctx.dtype)
        ops.token_shift(h, self.mu, cache.block_state, shifted, ctx.token_seq, ctx.seq_start, ctx.seq_slots, N)
        pending = NormedBranch(self.mixer.forward(shifted, ctx, cache), self.norms[1])
        if self.feed_forward is not None:
            normed = ctx.scratch.get("block.normed", (N, H), ctx.dtype)
            self._settle(residual, pending, self.norms[2], normed)
            pending = NormedBranch(self.feed_forward.forward(normed, ctx), self.norms[3])
        if self.side:
            sd = self.side
            rounded = ctx.scratch.get("block.normed", (N, H), ctx.dtype)
            self._settle(residual, pending, "round", rounded)
            a = ctx.scratch.get("side.a", (N, sd["dim"]), ctx.dtype)
            linear(rounded, self.w_side_gate, a)
            g = ctx.scratch.get("side.g", (N, sd["dim"]), ctx.dtype)
            ops.side_gate(a, ctx.token_ids, self.side_table, g, sd["index"] * sd["dim"])
            y = ctx.scratch.get("side.out", (N, H), ctx.dtype)
            pending = NormedBranch(linear(g, self.w_side_proj, y), self.side_norm)
        return residual, pending

    def finish(self, residual, pending, final_norm, ctx, out, normalize: bool = True):
        """out[r] = final_norm(stream + pending) of wanted row r (the pending sum is done in registers for those rows
        only: nothing reads the stream after the tail)."""
        from ..csrc import ops
        if ctx.want_all:
            return self._settle(residual, pending, final_norm if normalize else "round", out)
        return ops.settle_norm(residual, pending.branch if pending else None, pending.norm if pending else None,
                               final_norm if normalize else "round", out, rows=ctx.want_rows[:ctx.n_want], n_rows=ctx.n_want,
                               compute_dtype=ctx.dtype)


class HyperPending:
    """A sublayer's output (compute type) that is still to be added to the streams: every stream becomes a mix of the
    old streams plus its share of the output."""

    def __init__(self, branch, mix, out_coef):
        self.branch, self.mix, self.out_coef = branch, mix, out_coef


class HyperConnectionBlock(Part):
    """Pre-norm sublayers on a hidden state of `streams` copies per token ([N, streams * hidden], float32).  For
    sublayer q (1: mixer, 2: feed-forward) with the tensors `hc<q>.in` [s], `hc<q>.out` [s], `hc<q>.mix` [s, s]
    (indexed [from, to]):

        u = sum_s in[s] x_s;   y = sublayer(norm(u));   x_to <- sum_from mix[from, to] x_from + mult * out[to] * y

    `streams=None` is the plain residual sum x <- x + mult * y on one stream, without those tensors.  The sum is left
    pending and settled by whoever reads the streams next, in the kernel that forms and normalises its own input,
    so a sublayer costs one pass over the streams.  `finish` is the model's tail: the sum of the streams of the
    wanted rows, normalised."""
    stream_dtype = "float32"

    def __init__(self, mixer, feed_forward, norm: PartSpec, hidden_size: int, streams=None, residual_mult: float = 1.0,
                 names=("norm1", "norm2"), connection_names=("hc1.", "hc2.")):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.hidden_size, self.streams, self.mult = int(hidden_size), streams, float(residual_mult)
        self.n_streams = int(streams or 1)
        self.names, self.connection_names = tuple(names), tuple(connection_names)
        self.norms = [build_part("norm", norm) for _ in range(2 if feed_forward is not None else 1)]
        self.coef = []                 # per sublayer: (in [s], mult * out [s], mix [s, s]) float32

    def weight_specs(self, prefix: str) -> dict:
        from ..weights.loader import WeightSpec
        specs, s = {}, self.n_streams
        for part, name in zip(self.norms, self.names):
            specs.update(part.weight_specs(prefix + name))
        if self.streams is not None:
            for c in self.connection_names[:len(self.norms)]:
                specs.update({prefix + c + "in": WeightSpec((s,), "bias"), prefix + c + "out": WeightSpec((s,), "bias"),
                              prefix + c + "mix": WeightSpec((s, s), "bias")})
        specs.update(self.mixer.weight_specs(prefix))
        if self.feed_forward is not None:
            specs.update(self.feed_forward.weight_specs(prefix))
        return specs

    def ignorable(self, prefix: str):
        """Names that a checkpoint may hold although this block does not read them: the norm and connection tensors of
        a feed-forward the layer does not have."""
        if self.feed_forward is not None or len(self.names) < 2:
            return []
        c = self.connection_names[1] if len(self.connection_names) > 1 else None
        return [prefix + self.names[1]] + ([prefix + c + k for k in ("in", "out", "mix")] if c else [])

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        import torch
        for part, name in zip(self.norms, self.names):
            part.bind(weights, prefix + name, dtype, device)
        self.coef = []
        if self.streams is not None:
            raw = [[weights[prefix + c + k] for k in ("in", "out", "mix")] for c in self.connection_names[:len(self.norms)]]
            getattr(weights, "wait", lambda: None)()          # a streamed checkpoint: the tensors are in place now
            for into, out, mix in raw:
                f = dict(device=device, dtype=torch.float32)
                self.coef.append((into.to(**f).contiguous(), (out.to(**f) * self.mult).contiguous(), mix.to(**f).contiguous()))
        else:
            one = torch.ones(1, dtype=torch.float32, device=device)
            self.coef = [(one, one * self.mult, one.view(1, 1))] * len(self.norms)
        self.mixer.bind(weights, prefix, dtype, device)
        if self.feed_forward is not None:
            self.feed_forward.bind(weights, prefix, dtype, device)

    def _read(self, residual, pending, which: int, ctx):
        """Settle `pending` and return the normalised input of sublayer `which`."""
        from ..csrc import ops
        if pending is not None and not isinstance(pending, HyperPending):
            raise TypeError("streams take a HyperPending as their pending sum")
        normed = ctx.scratch.get("block.normed", (residual.shape[0], self.hidden_size), ctx.dtype)
        norm = self.norms[which]
        return ops.hyper_norm(residual, self.n_streams, pending.branch if pending else None, pending.mix if pending else None,
                              pending.out_coef if pending else None, self.coef[which][0], norm.weight, norm.eps, normed)

    def forward(self, residual, delta, ctx, cache):
        normed = self._read(residual, delta, 0, ctx)
        pending = HyperPending(self.mixer.forward(normed, ctx, cache), self.coef[0][2], self.coef[0][1])
        if self.feed_forward is None:
            return residual, pending
        normed = self._read(residual, pending, 1, ctx)
        return residual, HyperPending(self.feed_forward.forward(normed, ctx), self.coef[1][2], self.coef[1][1])

    def finish(self, residual, pending, final_norm, ctx, out, normalize: bool = True):
        """out[r] = norm(sum of the streams of wanted row r) with the pending sum settled on the way (for these rows
        only, in registers: nothing reads the streams after the tail).  `normalize=False`: the plain sum."""
        from ..csrc import ops
        rows = None if ctx.want_all else ctx.want_rows[:ctx.n_want]
        dtype = pending.branch.dtype if pending is not None else ctx.dtype
        return ops.hyper_norm(residual, self.n_streams, pending.branch if pending else None, pending.mix if pending else None,
                              pending.out_coef if pending else None, None, final_norm.weight, final_norm.eps, out, rows=rows,
                              n_rows=ctx.n_want, normalize=normalize, compute_dtype=dtype)


register_part("block", "hyper_connections", HyperConnectionBlock)
register_part("block", "pre_norm", PreNormBlock)
register_part("block", "sandwich_norm", SandwichNormBlock)
register_part("block", "shift_sandwich", ShiftSandwichBlock)
