"""How a layer's parts are arranged."""
from __future__ import annotations

import os
from typing import Dict, List

import torch

from ..config.specs import LayerSpec
from ..profile import scope
from ..weights.decl import TensorDecl
from .base import (BuildEnv, DeferredNorm, NormedRows, ResidualSink, RoutedRows, ShiftedRows, build_feed_forward, build_mixer,
                   build_norm, register_arrangement)


# From this many tokens in a step a part is offered to add into the residual itself (the products of
# fewer rows are split over K or run as kernels without that epilogue).
ADD_INTO_MIN_TOKENS = 256


def _is_partial_sums(x, n_rows: int) -> bool:
    """float32 [S, >= n_rows, H], contiguous: the form in which a norm's kernel adds a result into the stream."""
    return isinstance(x, torch.Tensor) and x.dim() == 3 and x.dtype == torch.float32 and x.is_contiguous() \
        and x.shape[1] >= n_rows


@register_arrangement("pre_norm")
class PreNormBlock:
    """x += mixer(norm1(x)); x += ff(norm2(x)) (rocml/src/forward/mod.rs:281-340).

    The additions are not done here: each part's result travels on as a *delta*, and the
    next norm adds it into the 32-bit residual stream in the same kernel that normalises.
    ``forward`` therefore takes the delta still pending from the layer before and returns
    its own feed-forward's delta."""

    def __init__(self, spec: LayerSpec, hidden: int, env: BuildEnv, mixer_spec=None):
        self.spec = spec
        self.prefix = spec.prefix
        self.mixer_norm = build_norm(spec.mixer_norm, hidden, env)
        self.mixer = build_mixer(mixer_spec or spec.mixer, hidden, env)
        self.ff_norm = build_norm(spec.ff_norm, hidden, env)
        self.ff = build_feed_forward(spec.feed_forward, hidden, env)

    # The four parts' tensor-name prefixes, as the layer's spec gives them.
    def _names(self):
        p, s = self.prefix, self.spec
        return (f"{p}.{s.mixer_norm_name}", f"{p}.{s.mixer_name}", f"{p}.{s.ff_norm_name}", f"{p}.{s.ff_name}")

    def declare(self) -> List[TensorDecl]:
        n1, mx, n2, ff = self._names()
        return self.mixer_norm.declare(n1) + self.mixer.declare(mx) + self.ff_norm.declare(n2) + self.ff.declare(ff)

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n1, mx, n2, ff = self._names()
        self.mixer_norm.load(tensors, n1)
        self.mixer.load(tensors, mx)
        self.ff_norm.load(tensors, n2)
        self.ff.load(tensors, ff)

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for p in (self.mixer_norm, self.mixer, self.ff_norm, self.ff))

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in (self.mixer_norm, self.mixer, self.ff_norm, self.ff))

    def workspace_bytes(self, n_tokens: int) -> int:
        """Each half of the layer holds its norm's rows and its part's buffers; the halves follow one another."""
        return max(self.mixer_norm.workspace_bytes(n_tokens) + self.mixer.workspace_bytes(n_tokens),
                   self.ff_norm.workspace_bytes(n_tokens) + self.ff.workspace_bytes(n_tokens))

    def cost(self, q_lens, kv_lens):
        parts = [p.cost(q_lens, kv_lens) for p in (self.mixer_norm, self.mixer, self.ff_norm, self.ff)]
        return sum(p[0] for p in parts), sum(p[1] for p in parts)

    chains = True          # forward() accepts next_block (see below)

    def forward(self, resid, pending, batch, view, next_block=None):
        """``pending`` is what the layer before left: a delta, or a DeferredNorm when it has added its
        result into the residual itself and prepared this layer's first norm.  For a decode step of
        up to 16 tokens the parts are offered to do the same for the norm that follows them
        (ResidualSink), when the part after that norm can take the deferred rows: the norm kernels
        then disappear from the step.  RB_DEFER=0 turns the offers off (and those to prompts, below)."""
        T = batch.n_tokens
        offers = batch.is_decode and T <= 16 and _defer_enabled()     # beyond 16 tokens the norm kernels are cheaper (measured)
        # Prompts: a part may be told to add its result into the residual itself (``add_into``; it then
        # returns None, nothing is pending, and the following norm only normalises): the delta of a
        # few thousand rows then never goes through memory.  Parts that set ``can_add_into`` get the offer.
        adds = not batch.is_decode and T > ADD_INTO_MIN_TOKENS and _defer_enabled()
        with scope(op="mixer_norm"):
            xn = self.mixer_norm.forward(resid, pending, T)
        if offers and getattr(self.mixer, "can_sink", False) and _takes(self.ff, batch):
            delta = self.mixer.forward(xn, batch, view, sink=ResidualSink(resid, self.ff_norm))
        elif adds and getattr(self.mixer, "can_add_into", False):
            delta = self.mixer.forward(xn, batch, view, add_into=resid)
        else:
            delta = self.mixer.forward(xn, batch, view)
        with scope(op="ff_norm"):
            xn = self.ff_norm.forward(resid, delta, T)
        nxt = getattr(next_block, "mixer", None)
        if offers and nxt is not None and getattr(self.ff, "can_sink", False) and _takes(nxt, batch):
            return self.ff.forward(xn, batch, sink=ResidualSink(resid, next_block.mixer_norm))
        if adds and getattr(self.ff, "can_add_into", False):
            return self.ff.forward(xn, batch, add_into=resid)
        return self.ff.forward(xn, batch)


def _takes(part, batch) -> bool:
    f = getattr(part, "takes_deferred", None)
    return bool(f(batch)) if f is not None else False


def _defer_enabled() -> bool:
    return os.environ.get("RB_DEFER", "1") != "0"


@register_arrangement("sandwich_norm")
class SandwichNormBlock:
    """x += post1(mixer(norm1(x))); x += post2(ff(norm2(x))): a norm before and after each sublayer.

    A sublayer's result (a delta, possibly as partial sums) is normalised on its own before it joins the
    residual stream, so it cannot ride along to the next norm as a pre-norm block's delta does.  One
    kernel adds the partial sums, normalises them, adds into the 32-bit residual and normalises that for
    the sublayer that follows: after the mixer the feed-forward's norm, after the feed-forward the first norm
    of the block that follows when that is a block of this kind (it gets the rows as ``NormedRows``).  A routed
    feed-forward's weighted sum over a token's experts happens in the same kernel.  Nothing is left pending.
    A layer without a feed-forward has only the first half."""

    chains = True          # forward() accepts next_block

    def __init__(self, spec: LayerSpec, hidden: int, env: BuildEnv, mixer_spec=None):
        if spec.mixer_post_norm is None or (spec.feed_forward is not None and spec.ff_post_norm is None):
            from ..errors import ConfigError
            raise ConfigError("a sandwich_norm layer needs a post norm for each of its sublayers")
        self.spec = spec
        self.prefix = spec.prefix
        self.env = env
        self.hidden = hidden
        self.mixer_norm = build_norm(spec.mixer_norm, hidden, env)
        self.mixer = build_mixer(mixer_spec or spec.mixer, hidden, env)
        self.mixer_post = build_norm(spec.mixer_post_norm, hidden, env)
        self.ff = self.ff_norm = self.ff_post = None
        if spec.feed_forward is not None:
            self.ff_norm = build_norm(spec.ff_norm, hidden, env)
            self.ff = build_feed_forward(spec.feed_forward, hidden, env)
            self.ff_post = build_norm(spec.ff_post_norm, hidden, env)

    def _parts(self):
        p, s = self.prefix, self.spec
        out = [(self.mixer_norm, f"{p}.{s.mixer_norm_name}"), (self.mixer, f"{p}.{s.mixer_name}"),
               (self.mixer_post, f"{p}.{s.mixer_post_norm_name}")]
        if self.ff is not None:
            out += [(self.ff_norm, f"{p}.{s.ff_norm_name}"), (self.ff, f"{p}.{s.ff_name}"),
                    (self.ff_post, f"{p}.{s.ff_post_norm_name}")]
        return out

    def declare(self) -> List[TensorDecl]:
        return [d for part, name in self._parts() for d in part.declare(name)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for part, name in self._parts():
            part.load(tensors, name)

    @property
    def graph_safe(self) -> bool:
        return all(part.graph_safe for part, _ in self._parts())

    def weight_bytes(self) -> int:
        return sum(part.weight_bytes() for part, _ in self._parts())

    def workspace_bytes(self, n_tokens: int) -> int:
        half1 = self.mixer_norm.workspace_bytes(n_tokens) + self.mixer.workspace_bytes(n_tokens)
        half2 = 0 if self.ff is None else self.ff_norm.workspace_bytes(n_tokens) + self.ff.workspace_bytes(n_tokens)
        return max(half1, half2)

    def cost(self, q_lens, kv_lens):
        parts = [part.cost(q_lens, kv_lens) for part, _ in self._parts()]
        return sum(p[0] for p in parts), sum(p[1] for p in parts)

    def _post(self, resid, delta, post, nxt, T):
        """resid += post(delta); returns nxt(resid) when a norm follows."""
        from .. import kernels
        for n in (post, nxt):
            if n is not None and not hasattr(n, "weight"):
                raise NotImplementedError("sandwich_norm is built for norms with a weight vector and an eps (rmsnorm)")
        out = None
        if nxt is not None:
            out = torch.empty((T, self.hidden), dtype=self.env.act_dtype, device=resid.device)
        w_next, eps_next = (nxt.weight, nxt.eps) if nxt is not None else (None, 0.0)
        if isinstance(delta, RoutedRows):
            kernels.postnorm_add_norm(resid, delta.rows, post.weight, post.eps, w_next, eps_next, out,
                                      row_of=delta.row_of, weights=delta.weights, top=delta.top)
        else:
            kernels.postnorm_add_norm(resid, delta, post.weight, post.eps, w_next, eps_next, out)
        return out

    def forward(self, resid, pending, batch, view, next_block=None):
        T = batch.n_tokens
        if isinstance(pending, NormedRows) and pending.norm is self.mixer_norm:
            xn = pending.x                                       # the block before has run this block's first norm
        else:
            with scope(op="mixer_norm"):
                xn = self.mixer_norm.forward(resid, pending, T)  # (adds whatever a different kind of layer before left pending)
        delta = self.mixer.forward(xn, batch, view)
        # the norm that follows the last sublayer: the next block's first, when that block takes the rows
        after = next_block.mixer_norm if isinstance(next_block, SandwichNormBlock) and \
            hasattr(next_block.mixer_norm, "weight") and next_block.mixer_norm.weight is not None and \
            next_block.mixer_norm.weight.dtype == self.mixer_post.weight.dtype else None
        with scope(op="mixer_post_norm"):
            xn = self._post(resid, delta, self.mixer_post, self.ff_norm if self.ff is not None else after, T)
        if self.ff is None:
            return self._handed(xn, after, resid)
        if getattr(self.ff, "sums_later", False):
            delta = self.ff.forward(xn, batch, sum_later=True)
        else:
            delta = self.ff.forward(xn, batch)
        with scope(op="ff_post_norm"):
            xn = self._post(resid, delta, self.ff_post, after, T)
        return self._handed(xn, after, resid)

    def _handed(self, rows, norm, resid):
        if norm is None:
            return None
        return NormedRows(rows, None, norm.eps, self.hidden, norm, resid)


@register_arrangement("parallel")
class ParallelBlock:
    """h = norm(x); x += mixer(h) + ff(h): one norm, and both sublayers read its output.

    Both results travel as deltas (partial sums over K) and ride on, as a pair, to the next layer's norm (or the
    model's last one), which adds the mixer's and then the feed-forward's in the kernel that normalises; a result
    in another form joins the 32-bit residual stream in a small kernel of its own.  For prompts the sublayers are offered to add into the residual
    inside their last product instead.  A layer without a feed-forward has only the mixer."""

    chains = False

    def __init__(self, spec: LayerSpec, hidden: int, env: BuildEnv, mixer_spec=None):
        self.spec = spec
        self.prefix = spec.prefix
        self.norm = build_norm(spec.mixer_norm, hidden, env)
        self.mixer = build_mixer(mixer_spec or spec.mixer, hidden, env)
        self.ff = build_feed_forward(spec.feed_forward, hidden, env) if spec.feed_forward is not None else None
        self.mixer_norm = self.norm        # the name other arrangements look for in the block after them

    def _parts(self):
        p, s = self.prefix, self.spec
        out = [(self.norm, f"{p}.{s.mixer_norm_name}"), (self.mixer, f"{p}.{s.mixer_name}")]
        if self.ff is not None:
            out.append((self.ff, f"{p}.{s.ff_name}"))
        return out

    def declare(self) -> List[TensorDecl]:
        return [d for part, name in self._parts() for d in part.declare(name)]

    def ignorable(self) -> List[str]:
        return [n for part, name in self._parts() for n in getattr(part, "ignorable", lambda prefix: [])(name)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for part, name in self._parts():
            part.load(tensors, name)

    @property
    def graph_safe(self) -> bool:
        return all(part.graph_safe for part, _ in self._parts())

    def weight_bytes(self) -> int:
        return sum(part.weight_bytes() for part, _ in self._parts())

    def workspace_bytes(self, n_tokens: int) -> int:
        """The norm's rows live through both sublayers, and the mixer's delta until the feed-forward is done."""
        return self.norm.workspace_bytes(n_tokens) + self.mixer.workspace_bytes(n_tokens) + \
            (self.ff.workspace_bytes(n_tokens) if self.ff is not None else 0)

    def cost(self, q_lens, kv_lens):
        parts = [part.cost(q_lens, kv_lens) for part, _ in self._parts()]
        return sum(p[0] for p in parts), sum(p[1] for p in parts)

    def _normed(self, resid, pending, T):
        """(the mixer's input, the feed-forward's input): here the same rows."""
        with scope(op="mixer_norm"):
            xn = self.norm.forward(resid, pending, T)        # adds what the layer before left, then normalises
        if isinstance(xn, DeferredNorm):
            xn = xn.materialize()
        return xn, xn

    def forward(self, resid, pending, batch, view):
        from .. import kernels
        T = batch.n_tokens
        adds = not batch.is_decode and T > ADD_INTO_MIN_TOKENS and _defer_enabled()
        xn, xf = self._normed(resid, pending, T)
        # Both sublayers read the stream as it was before either: with the offer to add into the stream inside
        # their last product, the feed-forward's input is formed before the mixer adds.
        if adds and getattr(self.mixer, "can_add_into", False):
            delta = self.mixer.forward(xn, batch, view, add_into=resid)
        else:
            delta = self.mixer.forward(xn, batch, view)
        if self.ff is None:
            return delta
        if adds and getattr(self.ff, "can_add_into", False):
            if delta is not None:
                with scope(op="mixer_add"):
                    kernels.residual_inject(resid, delta)
            return self.ff.forward(xf, batch, add_into=resid)
        ff_delta = self.ff.forward(xf, batch)
        if delta is None:
            return ff_delta
        if _is_partial_sums(delta, T) and _is_partial_sums(ff_delta, T):
            return (delta, ff_delta)          # the next norm adds both, the mixer's first: no kernel for the sum
        with scope(op="mixer_add"):
            kernels.residual_inject(resid, delta)
        return ff_delta


@register_arrangement("parallel_two_norms")
class ParallelTwoNormsBlock(ParallelBlock):
    """x += mixer(norm1(x)) + ff(norm2(x)): the parallel layer with a norm for each sublayer, both of the same x.

    Two norms of one row with one eps share the row's statistics and differ by their weights, so one kernel adds
    what the layer before left pending, and writes both sublayers' inputs.  Everything else is the parallel layer."""

    def __init__(self, spec: LayerSpec, hidden: int, env: BuildEnv, mixer_spec=None):
        super().__init__(spec, hidden, env, mixer_spec)
        self.ff_norm = build_norm(spec.ff_norm, hidden, env) if self.ff is not None else None

    def _parts(self):
        out = super()._parts()
        if self.ff_norm is not None:
            out.insert(1, (self.ff_norm, f"{self.prefix}.{self.spec.ff_norm_name}"))
        return out

    def workspace_bytes(self, n_tokens: int) -> int:
        return super().workspace_bytes(n_tokens) + (self.ff_norm.workspace_bytes(n_tokens) if self.ff_norm is not None else 0)

    def _normed(self, resid, pending, T):
        if self.ff_norm is None:
            return super()._normed(resid, pending, T)
        with scope(op="mixer_norm"):
            if hasattr(self.norm, "forward_with"):
                return self.norm.forward_with(self.ff_norm, resid, pending, T)
            xn = self.norm.forward(resid, pending, T)
            if isinstance(xn, DeferredNorm):
                xn = xn.materialize()
            return xn, self.ff_norm.forward(resid, None, T)


POST_NORM_NAMES = {"mixer_scale": "mixer_scale", "ff_scale": "ff_scale", "shift": "shift"}


@register_arrangement("post_norm")
class PostNormBlock:
    """x <- norm1(alpha x + g1 * mixer(h)); x <- norm2(alpha x + g2 * ff(x)): the norm follows the sum, so the 32-bit
    stream IS the normalised row and the sublayers read it as it is.

    Parameters (``LayerSpec.arrangement_params``): ``alpha``, the factor on the stream inside the sum; ``layer_scale``:
    each sublayer's result is multiplied, element by element, by a vector of the layer before it joins the sum;
    ``token_shift``: the mixer reads h_t = x_t + (x_(t-1) - x_t) * mu instead of x_t, mu a vector of the layer and
    x_(t-1) the row of the token before in the same sequence (zeros before the first); the last row of every step
    is kept per sequence, as a state of the layer beside whatever its mixer keeps (``cache_requirement``).

    One kernel does a sublayer's sum and norm (``kernels.postln``): it adds the result's partial sums in their order,
    applies the vector, alpha and the norm in 32-bit, writes the stream in place and, when a product reads the row
    next, the row in the activations' type as well.  One kernel blends the rows for the mixer and hands the
    kept row over; in a step of one token a sequence the layer's LAST sum-and-norm kernel does that for the layer after
    it (``ShiftedRows``), whose row before is then always the one its slot kept.  Nothing else is left pending for the
    layer after it.  A layer without a feed-forward has only the first half."""

    chains = True              # forward() accepts next_block
    wants_next_view = True     # ... and next_view, the cache view of the run that follows

    def __init__(self, spec: LayerSpec, hidden: int, env: BuildEnv, mixer_spec=None):
        from ..config.specs import tensor_names
        from ..errors import ConfigError
        p = spec.arrangement_params
        unknown = sorted(set(p) - {"alpha", "layer_scale", "token_shift", "names"})
        if unknown:
            raise ConfigError(f"post_norm: unknown parameters {unknown}")
        self.spec = spec
        self.prefix = spec.prefix
        self.env = env
        self.hidden = hidden
        self.alpha = float(p.get("alpha", 1.0))
        self.layer_scale = bool(p.get("layer_scale", False))
        self.token_shift = bool(p.get("token_shift", False))
        try:
            self.names = tensor_names(p, POST_NORM_NAMES)
        except ValueError as e:
            raise ConfigError(f"post_norm: {e}") from None
        self.mixer_norm = build_norm(spec.mixer_norm, hidden, env)
        self.mixer = build_mixer(mixer_spec or spec.mixer, hidden, env)
        self.ff = self.ff_norm = None
        if spec.feed_forward is not None:
            self.ff_norm = build_norm(spec.ff_norm, hidden, env)
            self.ff = build_feed_forward(spec.feed_forward, hidden, env)
        for n in (self.mixer_norm, self.ff_norm):
            if n is not None and (not hasattr(n, "eps") or getattr(n, "offset", 0.0)):
                raise ConfigError("post_norm is built for norms with a plain weight vector and an eps (rmsnorm)")
        self.mixer_gain = self.ff_gain = self.mu = None
        self._w1 = self._w2 = None

    def _parts(self):
        p, s = self.prefix, self.spec
        out = [(self.mixer_norm, f"{p}.{s.mixer_norm_name}"), (self.mixer, f"{p}.{s.mixer_name}")]
        if self.ff is not None:
            out += [(self.ff_norm, f"{p}.{s.ff_norm_name}"), (self.ff, f"{p}.{s.ff_name}")]
        return out

    def _own(self):
        """(attribute, tensor name) of the arrangement's own vectors."""
        out = []
        if self.layer_scale:
            out.append(("mixer_gain", f"{self.prefix}.{self.names['mixer_scale']}.weight"))
            if self.ff is not None:
                out.append(("ff_gain", f"{self.prefix}.{self.names['ff_scale']}.weight"))
        if self.token_shift:
            out.append(("mu", f"{self.prefix}.{self.names['shift']}.weight"))
        return out

    def declare(self) -> List[TensorDecl]:
        return [d for part, name in self._parts() for d in part.declare(name)] + \
            [TensorDecl(name, (self.hidden,), "norm") for _, name in self._own()]

    def ignorable(self) -> List[str]:
        out = [n for part, name in self._parts() for n in getattr(part, "ignorable", lambda prefix: [])(name)]
        if self.ff is None:        # a layer without a feed-forward may still carry the second half's vectors
            out += [f"{self.prefix}.{self.spec.ff_norm_name}.weight", f"{self.prefix}.{self.names['ff_scale']}.weight"]
        return out

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for part, name in self._parts():
            part.load(tensors, name)
        for attr, name in self._own():
            setattr(self, attr, tensors[name].float().contiguous())      # 32-bit: they enter the stream's sum
        self._w1 = self.mixer_norm.weight.float().contiguous()
        self._w2 = self.ff_norm.weight.float().contiguous() if self.ff_norm is not None else None

    def cache_requirement(self):
        from ..cache.requirements import BundleRequirement, StateRequirement
        req = self.mixer.cache_requirement()
        if not self.token_shift:
            return req
        return BundleRequirement.of(req, shift=StateRequirement((self.hidden,), torch.float32))

    @property
    def graph_safe(self) -> bool:
        return all(part.graph_safe for part, _ in self._parts())

    def weight_bytes(self) -> int:
        own = sum(self.hidden * 4 for _ in self._own())
        return sum(part.weight_bytes() for part, _ in self._parts()) + own

    def workspace_bytes(self, n_tokens: int) -> int:
        esz = 4 if self.env.mode == "float32" else 2
        rows = n_tokens * self.hidden * esz
        return rows + max(self.mixer.workspace_bytes(n_tokens), self.ff.workspace_bytes(n_tokens) if self.ff is not None else 0)

    def cost(self, q_lens, kv_lens):
        parts = [part.cost(q_lens, kv_lens) for part, _ in self._parts()]
        return sum(p[0] for p in parts), sum(p[1] for p in parts)

    def _rows_for(self, resid, T):
        """The stream's rows as a product reads them: themselves in 32-bit mode, a copy in the activations' type otherwise."""
        from .. import kernels
        if self.env.act_dtype == torch.float32:
            return resid
        out = torch.empty((T, self.hidden), dtype=self.env.act_dtype, device=resid.device)
        kernels.cast(resid[:T], out)
        return out

    def _join(self, resid, pending):
        """Whatever a layer of another kind left pending joins the stream first."""
        from .. import kernels
        if pending is None or isinstance(pending, DeferredNorm):
            return
        for d in (pending if isinstance(pending, (tuple, list)) else (pending,)):
            if isinstance(d, RoutedRows):
                d = d.materialize()
            if d is not None:
                kernels.residual_inject(resid, d)

    def _next_shift(self, batch, next_block, next_view, resid):
        """(mu, kept rows, rows to fill) of the block that follows, when this block's last kernel can blend its input."""
        if not (batch.is_decode and isinstance(next_block, PostNormBlock) and next_block.token_shift and next_view is not None
                and "shift" in next_view.extras and next_block.hidden == self.hidden and next_block.env.act_dtype == self.env.act_dtype):
            return None, None, None
        out = torch.empty((batch.n_tokens, self.hidden), dtype=self.env.act_dtype, device=resid.device)
        return next_block.mu, next_view.extras["shift"].state, out

    def forward(self, resid, pending, batch, view, next_block=None, next_view=None):
        from .. import kernels
        T = batch.n_tokens
        act = self.env.act_dtype
        if isinstance(pending, ShiftedRows):
            h = pending.x if pending.block is self else None
            pending = None
        else:
            h = None
        self._join(resid, pending)
        n_mu, n_kept, n_out = self._next_shift(batch, next_block, next_view, resid)
        if h is not None and self.token_shift:
            pass                                    # the block before has blended this block's rows
        elif self.token_shift:
            h = torch.empty((T, self.hidden), dtype=act, device=resid.device)
            with scope(op="token_shift"):
                kernels.token_shift(resid, self.mu, view.extras["shift"].state, batch.seq_slot, batch.cu_q, batch.n_seqs,
                                    batch.max_q_len, h, T)
        else:
            with scope(op="mixer_input"):
                h = self._rows_for(resid, T)
        delta = self.mixer.forward(h, batch, view)
        delta = _as_partial_sums(delta, T)
        rows = None
        if self.ff is not None and act != torch.float32:
            rows = torch.empty((T, self.hidden), dtype=act, device=resid.device)
        last = self.ff is None
        with scope(op="mixer_post_norm"):
            kernels.postln(resid, delta, self.mixer_gain, self._w1, self.alpha, self.mixer_norm.eps, rows, batch.slot_of_token, T,
                           next_mu=n_mu if last else None, next_kept=n_kept if last else None, next_out=n_out if last else None)
        if not last:
            delta = _as_partial_sums(self.ff.forward(rows if rows is not None else resid, batch), T)
            with scope(op="ff_post_norm"):
                kernels.postln(resid, delta, self.ff_gain, self._w2, self.alpha, self.ff_norm.eps, None, batch.slot_of_token, T,
                               next_mu=n_mu, next_kept=n_kept, next_out=n_out)
        return ShiftedRows(n_out, next_block) if n_out is not None else None


def _as_partial_sums(delta, n_rows: int):
    """A sublayer's result in the form the sum's kernel adds: float32 [S, >= rows, H]."""
    if isinstance(delta, RoutedRows):
        delta = delta.materialize()
    if delta is None or _is_partial_sums(delta, n_rows):
        return delta
    if isinstance(delta, torch.Tensor) and delta.dim() == 2:
        delta = delta.unsqueeze(0)
    return delta.float().contiguous()
