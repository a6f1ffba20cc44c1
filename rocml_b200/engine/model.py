"""A decoder assembled from a ModelSpec: embedding, blocks, the order they run in, final
norm, head.  It is generic: the architecture lives in the spec, not here.

One forward pass (rocml/src/forward/mod.rs:271-378, chunk_forward.rs:97-188): embedding
gather into a 32-bit residual stream; the scheduled blocks; the final norm only on the rows
whose logits are wanted; the head on those rows -> float32 logits.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from ..profile import scope
from ..config.specs import MixerSpec, ModelSpec
from ..errors import ConfigError
from ..parts import BuildEnv, build_block, build_norm, build_position
from ..parts.linear import Linear
from ..weights.decl import TensorDecl
from ..weights.loader import load_tensors


class Model:
    def __init__(self, spec: ModelSpec, env: BuildEnv):
        self.spec = spec
        self.env = env
        self.hidden = spec.hidden
        self.vocab = spec.vocab
        readers = {e.layer for e in spec.schedule if e.reads_cache_of is not None}
        owners = {e.layer for e in spec.schedule if e.reads_cache_of is None}
        if readers & owners:
            raise ConfigError("a layer cannot both keep its own cache and read another's in one schedule")
        self.blocks = []
        for i, layer in enumerate(spec.layers):
            mixer_spec = layer.mixer
            if i in readers:
                mixer_spec = MixerSpec(mixer_spec.kind, tuple(sorted({**mixer_spec.params, "shares_cache": True}.items())),
                                       mixer_spec.position)
            self.blocks.append(build_block_with(layer, spec.hidden, env, mixer_spec))
        self.final_norm = build_norm(spec.final_norm, spec.hidden, env)
        # a norm of the embedding output: what enters the first layer, and the stream itself, is the normalised row
        self.embedding_norm = build_norm(spec.embedding_norm, spec.hidden, env) if spec.embedding_norm is not None else None
        self.head = Linear([spec.head_name[: -len(".weight")]], [spec.vocab], spec.hidden, False, env)
        self.embed: Optional[torch.Tensor] = None
        self.status: Optional[torch.Tensor] = None
        # a position vector added to the embedding output (its table of frequencies lives on the device)
        self.input_position = None
        if spec.input_position is not None and spec.input_position.kind != "none":
            self.input_position = build_position(spec.input_position, spec.hidden, env)
            if getattr(self.input_position, "width", None) != spec.hidden:
                raise ConfigError(f"position encoding {spec.input_position.kind!r} cannot be added to the embedding output")
        # tensors whose rows are added to the residual stream before some runs: name -> rows
        self.added_rows: Dict[str, int] = {}
        for e in spec.schedule:
            if e.add_row is not None:
                name, row, rows = e.add_row
                if not 0 <= row < rows or self.added_rows.setdefault(name, rows) != rows:
                    raise ConfigError(f"schedule: row {row} of {name!r} ({rows} rows) does not fit")
        self.added: Dict[str, torch.Tensor] = {}
        self.keeps_input = any(e.add_input for e in spec.schedule)

    # ---- tensors ------------------------------------------------------------------------------
    # Parts name their tensors '<stem>.weight'; the files of an architecture may append something else to
    # the stem, or nothing (``ModelSpec.weight_suffix``).  ``declare`` speaks the files' names, ``load``
    # takes them and hands the parts theirs.
    def _file_name(self, name: str) -> str:
        for ours, theirs in ((".weight", self.spec.weight_suffix), (".bias", self.spec.bias_suffix)):
            if theirs != ours and name.endswith(ours):
                return name[: -len(ours)] + theirs
        return name

    def _declare_parts(self) -> List[TensorDecl]:
        out = [TensorDecl(self.spec.embedding_name, (self.vocab, self.hidden), "matrix")]
        if self.embedding_norm is not None:
            out += self.embedding_norm.declare(self.spec.embedding_norm_name[: -len(".weight")])
        for name, rows in self.added_rows.items():
            out.append(TensorDecl(name, (rows, self.hidden), "matrix"))
        for b in self.blocks:
            out += b.declare()
        out += self.final_norm.declare(self.spec.final_norm_name[: -len(".weight")])
        if not self.spec.tie_embeddings:
            out += self.head.declare("")
        return out

    def declare(self) -> List[TensorDecl]:
        return [TensorDecl(self._file_name(d.name), d.shape, d.role) for d in self._declare_parts()]

    def ignorable(self) -> List[str]:
        """Tensors a folder may hold that the model does not read: a stored head when the
        head is tied to the embedding."""
        out = [self.spec.head_name] if self.spec.tie_embeddings else []
        for b in self.blocks:
            out += getattr(b, "ignorable", lambda: [])()
        return [self._file_name(n) for n in out]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        if self.spec.weight_suffix != ".weight" or self.spec.bias_suffix != ".bias":
            tensors = {d.name: tensors[self._file_name(d.name)] for d in self._declare_parts()}
        self.embed = tensors[self.spec.embedding_name]
        if self.embedding_norm is not None:
            self.embedding_norm.load(tensors, self.spec.embedding_norm_name[: -len(".weight")])
        self.added = {name: tensors[name] for name in self.added_rows}
        for b in self.blocks:
            b.load(tensors)
        self.final_norm.load(tensors, self.spec.final_norm_name[: -len(".weight")])
        if self.spec.tie_embeddings:
            self.head.adopt(self.embed)
        else:
            self.head.load(tensors, "")
        self.status = torch.zeros(1, dtype=torch.int32, device=self.env.device)

    def load_folder(self, folder: str) -> None:
        self.load(load_tensors(folder, self.declare(), self.env.mode, self.env.device, self.ignorable()))

    def load_random(self, seed: int) -> None:
        """Random weights made directly on the device (the distributions of the random-weights
        mode; no folder is written)."""
        from ..weights.random_init import random_tensor
        dt = torch.float32 if self.env.mode == "float32" else torch.bfloat16
        tensors = {}
        for d in self.declare():
            t = random_tensor(d, seed, self.env.device, torch.bfloat16)
            tensors[d.name] = t if d.role == "int_table" else t.to(dt)
        self.load(tensors)

    # ---- facts ----------------------------------------------------------------------------------
    @property
    def graph_safe(self) -> bool:
        return all(b.graph_safe for b in self.blocks) and self.final_norm.graph_safe and \
            (self.embedding_norm is None or self.embedding_norm.graph_safe)

    def cache_requirements(self):
        # an arrangement that keeps something of its own a sequence (the row of the token before) answers for its layer
        return [getattr(self.blocks[e.layer], "cache_requirement", self.blocks[e.layer].mixer.cache_requirement)()
                for e in self.spec.schedule]

    def reads_cache_of(self):
        return [e.reads_cache_of for e in self.spec.schedule]

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights a step reads once: every scheduled block, the final norm, the head
        (the embedding rows it gathers are negligible)."""
        n = sum(self.blocks[e.layer].weight_bytes() for e in self.spec.schedule)
        return n + self.final_norm.weight_bytes() + self.head.weight_bytes()

    def workspace_bytes(self, n_tokens: int, n_want: int) -> int:
        """Device memory a step of ``n_tokens`` tokens allocates besides weights and cache: the 32-bit
        residual stream, the widest layer's buffers (asked of the parts: layers run one after another,
        and a delta outlives its layer by one norm), and float32 logits for ``n_want`` rows."""
        widest = max([getattr(b, "workspace_bytes", lambda n: 0)(n_tokens) for b in self.blocks] or [0])
        return n_tokens * self.hidden * 4 * 2 + 2 * widest + n_want * (self.vocab * 4 + self.hidden * 4)

    def step_cost(self, q_lens, kv_lens, n_want: int):
        """(bytes, floating-point operations) a step has to move and do at least: every scheduled
        block's weights once and its products and attention over the given sequences (``q_lens`` new
        tokens each, ``kv_lens`` long afterwards, whose keys and values are read once), the final norm,
        and the head on ``n_want`` rows.  Asked of the parts, so it holds for any arrangement."""
        nbytes = flops = 0
        for e in self.spec.schedule:
            block = self.blocks[e.layer]
            if hasattr(block, "cost"):
                b, f = block.cost(q_lens, kv_lens)
            else:
                b, f = block.weight_bytes(), 0
            nbytes, flops = nbytes + b, flops + f
        hb, hf = self.head.cost(n_want)
        nb = self.embedding_norm.weight_bytes() if self.embedding_norm is not None else 0
        return nbytes + self.final_norm.weight_bytes() + nb + hb, flops + hf

    # ---- the pass ---------------------------------------------------------------------------------
    def forward(self, batch, cache) -> Optional[torch.Tensor]:
        T = batch.n_tokens
        resid = torch.empty((T, self.hidden), dtype=torch.float32, device=self.env.device)
        x0 = torch.empty_like(resid) if self.keeps_input else None
        # with a norm of the embedding output the gathered rows land beside the stream, and the norm writes the stream
        rows = torch.empty_like(resid) if self.embedding_norm is not None else resid
        with scope(op="embedding"):
            if self.input_position is None and self.spec.embedding_scale == 1.0 and (x0 is None or rows is not resid):
                kernels.embedding(batch.token_ids, self.embed, rows, self.status)
            else:
                kernels.embedding_pos(batch.token_ids, self.embed, rows, self.spec.embedding_scale, batch.positions,
                                      self.input_position.inv_freq if self.input_position is not None else None,
                                      copy=x0 if rows is resid else None, status=self.status)
        if self.embedding_norm is not None:
            with scope(op="embedding_norm"):
                kernels.add_rmsnorm(rows, None, self.embedding_norm.weight, self.embedding_norm.eps, resid, n_rows=T,
                                    write_back=False)
                if x0 is not None:
                    x0.copy_(resid)
        pending = None
        sched = self.spec.schedule
        for i, e in enumerate(sched):
            block = self.blocks[e.layer]
            if e.add_input or e.add_row is not None:
                # what the layer before left pending joins the stream first, then the embedding output, then the row
                with scope(layer=i, op="stream_additions"):
                    if isinstance(pending, (tuple, list)):          # a pair of results: the first joins alone
                        kernels.residual_inject(resid, pending[0])
                        pending = pending[1]
                    delta = pending if isinstance(pending, torch.Tensor) else None
                    vec = self.added[e.add_row[0]][e.add_row[1]] if e.add_row is not None else None
                    kernels.residual_inject(resid, delta, x0 if e.add_input else None, vec)
                pending = None
            with scope(layer=i):
                if getattr(block, "chains", False):
                    # a block may prepare the first norm of the block that follows it
                    # (not across additions to the stream: they come before that norm)
                    nxt = self.blocks[sched[i + 1].layer] if i + 1 < len(sched) and not sched[i + 1].add_input \
                        and sched[i + 1].add_row is None else None
                    if getattr(block, "wants_next_view", False):
                        pending = block.forward(resid, pending, batch, cache.views[i], next_block=nxt,
                                                next_view=cache.views[i + 1] if nxt is not None else None)
                    else:
                        pending = block.forward(resid, pending, batch, cache.views[i], next_block=nxt)
                else:
                    pending = block.forward(resid, pending, batch, cache.views[i])
        if batch.n_want == 0:
            return None
        with scope(op="final_norm"):
            xn = self.final_norm.forward(resid, pending, n_rows=batch.n_want, rows=batch.want_rows, write_back=False)
        logits = torch.empty((batch.n_want, self.vocab), dtype=torch.float32, device=self.env.device)
        self.head.forward(xn, logits, batch.n_want)
        if self.spec.logit_scale != 1.0:
            with scope(op="logit_scale"):
                kernels.scale_(logits, self.spec.logit_scale)
        return logits


def build_block_with(layer, hidden, env, mixer_spec):
    from ..parts.base import _lookup, _ARRANGEMENTS
    return _lookup(_ARRANGEMENTS, layer.arrangement, "arrangement")(layer, hidden, env, mixer_spec)


def declared_tensors(spec: ModelSpec) -> List[TensorDecl]:
    """The tensors a model of this spec reads from its folder (no device memory is touched)."""
    return Model(spec, BuildEnv(torch.device("cpu"), torch.bfloat16)).declare()
