"""Latent attention: keys and values of every head are unfolded from ONE cached vector a token.

    q = Wq h                    [heads, head_dim]
    c = rmsnorm(Wdown h) * w_c  [kv_rank]            the only thing the cache keeps
    k = Wuk c, v = Wuv c        head by head
    s_ij = (q_i . k_j) * scale over the causal window, softmax, o_i = sum_j a_ij v_j
    out = Wo concat_heads(gate_i * o_i),  gate = sigmoid(Wg h) per head (when ``gated``)

Computed without ever unfolding a cached token: (q . Wuk c) = (Wuk^T q) . c, so the queries are folded
into the latent space head by head (q' = Wuk_h^T q_h, [kv_rank]); the attention is then the
library's paged attention with ONE key/value head of size kv_rank whose keys and values are both the
cached latent; and the result per head, sum_j a_ij c_j, is unfolded with Wuv_h.  A decode step reads
kv_rank numbers a cached token instead of heads * (head_dim + v_head_dim).  No positions enter.

Two more parameters: ``q_rank``: the queries pass through a latent of their own, cq = rmsnorm(Wdq h) * w_q,
q = Wuq cq; ``rot_head_dim`` (with a rotate-half position encoding): every query head is [head_dim plain | rot
rotated] entries, Wdown h has kv_rank + rot rows of which the last rot, not normalised, are ONE rotated key part that
all heads share, and the score is (q_plain . k + q_rot . k_rot) * scale.  The cache then keeps [c | k_rot turned] a token
(padded with zeros to a multiple of 16); a folded query is [Wuk_h^T q_plain | q_rot turned], so the score is still one
dot product with the cached row; the values read the same rows, and the unfolding uses their first kv_rank entries.

One stacked product makes q | c | gate logits from the layer's input; one small kernel normalises the
latent into its page and writes the gates; two per-head products fold and unfold; the attention kernels
and the output product are the ones every attention layer uses.  Scores, softmax, the latent's norm and
the gates are 32-bit in both modes.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from .. import kernels
from ..cache.requirements import KVRequirement
from ..config.specs import MixerSpec, tensor_names
from ..errors import ConfigError
from ..profile import scope
from ..weights.decl import TensorDecl
from .attention import paged_attention
from .base import BuildEnv, DeferredNorm, Mixer, build_position, register_mixer
from .linear import Linear

TENSOR_NAMES = {"q": "q_proj", "down": "kv_down_proj", "latent_norm": "kv_norm", "up_k": "k_up_proj",
                "up_v": "v_up_proj", "gate": "gate_proj", "o": "o_proj", "q_down": "q_down_proj", "q_latent_norm": "q_norm"}


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, spec: MixerSpec, hidden: int, env: BuildEnv):
        p = spec.params
        self.env = env
        self.hidden = hidden
        self.heads = int(p["n_heads"])
        self.hd = int(p["head_dim"])
        self.vd = int(p.get("v_head_dim", self.hd))
        self.rank = int(p["kv_rank"])
        self.rot = int(p.get("rot_head_dim") or 0)
        self.q_rank = int(p["q_rank"]) if p.get("q_rank") else 0
        if min(self.heads, self.vd, self.rank) <= 0 or self.hd < 0 or self.rot < 0 or self.hd + self.rot <= 0:
            raise ConfigError("latent attention: heads, head sizes and the latent's size must be positive")
        # the width of a cached row: the latent alone, or the latent and the rotated key part padded to what the kernels take
        self.dp = self.rank if not self.rot else -(-(self.rank + self.rot) // 16) * 16
        if self.dp > 512:
            raise ConfigError(f"latent attention: a cached row of {self.dp} numbers is not supported (the attention "
                              "kernels take up to 512)")
        self.position = None
        if self.rot:
            if spec.position.kind != "rope_neox" or self.rot % 2:
                raise ConfigError("latent attention: the rotated part takes an even width and the rotate-half encoding")
            if not self.q_rank:
                raise ConfigError("latent attention: a rotated part without a query latent is not built")
            self.position = build_position(spec.position, self.rot, env)
            if self.position.rot_dim != self.rot:
                raise ConfigError("latent attention: the rotation must cover the whole rotated part")
        elif spec.position.kind != "none":
            raise ConfigError("latent attention: a position encoding needs rot_head_dim")
        if self.q_rank and not self.hd and not self.rot:
            raise ConfigError("latent attention: queries need a width")
        self.eps = float(p.get("latent_norm_eps", 1e-6))
        self.window = p.get("window")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.hd)
        self.gated = bool(p.get("gated", False))
        try:
            self.names = n = tensor_names(p, TENSOR_NAMES)
        except ValueError as e:
            raise ConfigError(f"latent attention: {e}") from None
        self.q_width = self.heads * (self.hd + self.rot)
        first = [n["q_down"], self.q_rank] if self.q_rank else [n["q"], self.q_width]
        stems = [first[0], n["down"]] + ([n["gate"]] if self.gated else [])
        outs = [first[1], self.rank + self.rot] + ([self.heads] if self.gated else [])
        self.proj = Linear(stems, outs, hidden, False, env)
        self.q_up = Linear([n["q"]], [self.q_width], self.q_rank, False, env) if self.q_rank else None
        self.q_latent_norm_w: Optional[torch.Tensor] = None
        self.o = Linear([n["o"]], [hidden], self.heads * self.vd, False, env)
        self.latent_norm_w: Optional[torch.Tensor] = None
        self.fold: Optional[torch.Tensor] = None       # [heads, kv_rank, head_dim]: Wuk_h^T
        self.unfold: Optional[torch.Tensor] = None     # [heads, v_head_dim, kv_rank]: Wuv_h

    def cache_requirement(self):
        return KVRequirement(1, self.dp, self.window, shared_values=True)

    def declare(self, prefix: str) -> List[TensorDecl]:
        n = self.names
        extra = []
        if self.q_rank:
            extra = self.q_up.declare(prefix) + [TensorDecl(f"{prefix}{n['q_latent_norm']}.weight", (self.q_rank,), "norm")]
        return self.proj.declare(prefix) + self.o.declare(prefix) + extra + [
            TensorDecl(f"{prefix}{n['latent_norm']}.weight", (self.rank,), "norm"),
            TensorDecl(f"{prefix}{n['up_k']}.weight", (self.heads * self.hd, self.rank), "matrix"),
            TensorDecl(f"{prefix}{n['up_v']}.weight", (self.heads * self.vd, self.rank), "matrix"),
        ]

    def load(self, tensors: Dict[str, torch.Tensor], prefix: str) -> None:
        n = self.names
        self.proj.load(tensors, prefix)
        self.proj.pad_rows(8)        # q | c | gates is rarely a multiple of 8 wide: the product's rows must start on 16 bytes
        self.o.load(tensors, prefix)
        self.latent_norm_w = tensors[f"{prefix}{n['latent_norm']}.weight"]
        if self.q_rank:
            self.q_up.load(tensors, prefix)
            self.q_latent_norm_w = tensors[f"{prefix}{n['q_latent_norm']}.weight"].float().contiguous()
            self.latent_norm_w = self.latent_norm_w.float().contiguous()      # the kernel of this form reads 32-bit vectors
        uk = tensors[f"{prefix}{n['up_k']}.weight"]
        uv = tensors[f"{prefix}{n['up_v']}.weight"]
        # per head: the key unfolding transposed (so that its product folds a query), the value unfolding as it is
        self.fold = uk.reshape(self.heads, self.hd, self.rank).transpose(1, 2).contiguous()
        self.unfold = uv.reshape(self.heads, self.vd, self.rank).contiguous()

    def weight_bytes(self) -> int:
        esz = 4 if self.env.mode == "float32" else 2
        return self.proj.weight_bytes() + self.o.weight_bytes() + self.heads * (self.hd + self.vd) * self.rank * esz + \
            (self.q_up.weight_bytes() if self.q_up is not None else 0)

    def workspace_bytes(self, n_tokens: int) -> int:
        esz = 4 if self.env.mode == "float32" else 2
        parts = 8 if n_tokens <= 128 else 1
        return n_tokens * (self.proj.n * max(esz, 4 * parts if parts > 1 else esz) + self.q_width * esz
                           + 2 * self.heads * self.rank * esz + self.heads * self.vd * esz + self.hidden * 4 * parts
                           + self.heads * 4 * (self.rank + 2) * (parts if parts > 1 else 0))

    def cost(self, q_lens, kv_lens):
        from ..profile import cost as C
        T = sum(q_lens)
        esz = 4 if self.env.mode == "float32" else 2
        fold = (self.heads * (self.hd + self.vd) * self.rank * esz, 2 * T * self.heads * (self.hd + self.vd) * self.rank)
        parts = [self.proj.cost(T), self.o.cost(T), fold,
                 C.attention(q_lens, kv_lens, self.heads, 1, self.dp, esz, int(self.window) if self.window else None)]
        if self.q_up is not None:
            parts.append(self.q_up.cost(T))
        # keys and values are one tensor: the attention's cost counts the cached bytes twice
        w = int(self.window) if self.window else 0
        shared = sum((kl - (max(0, kl - ql - w + 1) if w else 0)) * self.dp * esz
                     for ql, kl in zip(q_lens, kv_lens) if ql > 0 and kl > 0)
        return sum(p[0] for p in parts) - shared, sum(p[1] for p in parts)

    def forward(self, xn, batch, view):
        T = batch.n_tokens
        dev, act = self.env.device, self.env.act_dtype
        window = int(self.window) if self.window else 0
        if isinstance(xn, DeferredNorm):
            xn = xn.materialize()
        proj = self.proj.forward_auto(xn, T)              # [T, N] in the activations' type, or [S, T, N] float32 partial sums
        if self.q_rank:
            return self._forward_query_latent(proj, batch, view, window)
        q = None
        if proj.dim() == 3 or proj.dtype != act:
            q = torch.empty((T, self.q_width), dtype=act, device=dev)
        gates = torch.empty((T, self.heads), dtype=torch.float32, device=dev) if self.gated else None
        with scope(op="latent_norm_cache"):
            kernels.latent_prep(proj, T, self.q_width, self.rank, self.heads if self.gated else 0, self.latent_norm_w,
                                self.eps, q, gates, view.k, batch.positions, batch.slot_of_token, view.block_table)
        if q is None:
            q = proj[:, :self.q_width]
        folded = torch.empty((T, self.heads * self.rank), dtype=act, device=dev)
        with scope(op="fold_queries"):
            kernels.head_matmul(q, self.fold, folded, T)
        mixed = torch.empty((T, self.heads * self.rank), dtype=act, device=dev)
        paged_attention(folded, mixed, batch, view.k, view.v, view.block_table, self.heads, 1, self.rank, self.scale, window)
        attn = torch.empty((T, self.heads * self.vd), dtype=act, device=dev)
        with scope(op="unfold_values"):
            kernels.head_matmul(mixed, self.unfold, attn, T, row_scale=gates)
        return self.o.forward_delta(attn, T)

    def _forward_query_latent(self, proj, batch, view, window):
        """proj rows = [query latent | latent | rotated key part | gate logits]."""
        T = batch.n_tokens
        dev, act = self.env.device, self.env.act_dtype
        cos_sin = self.position.cos_sin(batch) if self.rot else None
        cq = torch.empty((T, self.q_rank), dtype=act, device=dev)
        gates = torch.empty((T, self.heads), dtype=torch.float32, device=dev) if self.gated else None
        with scope(op="latent_norm_cache"):
            kernels.latent_rot_prep(proj, T, self.q_rank, self.rank, self.rot, self.heads if self.gated else 0,
                                    self.q_latent_norm_w, self.latent_norm_w, self.eps, cq, gates, view.k, cos_sin,
                                    batch.positions, batch.slot_of_token, view.block_table)
        q = torch.empty((T, self.q_width), dtype=act, device=dev)
        self.q_up.forward(cq, q, T)
        per_head = self.hd + self.rot
        folded = (torch.empty if self.hd else torch.zeros)((T, self.heads * self.dp), dtype=act, device=dev)
        with scope(op="fold_queries"):
            if self.hd:
                kernels.head_matmul(q, self.fold, folded, T, x_group_stride=per_head, out_group_stride=self.dp)
            if self.dp > self.rank:
                kernels.latent_q_rot(q, self.heads, self.hd, self.rot, self.rank, cos_sin, folded, batch.slot_of_token, T)
        mixed = torch.empty((T, self.heads * self.dp), dtype=act, device=dev)
        paged_attention(folded, mixed, batch, view.k, view.v, view.block_table, self.heads, 1, self.dp, self.scale, window)
        attn = torch.empty((T, self.heads * self.vd), dtype=act, device=dev)
        with scope(op="unfold_values"):
            kernels.head_matmul(mixed, self.unfold, attn, T, row_scale=gates, x_group_stride=self.dp)
        return self.o.forward_delta(attn, T)
