"""Grouped-query softmax attention over the paged cache.

Order, as in the reference (rocml/src/forward/attention.rs:56-244, attention_chunk.rs:
75-325): q, k, v projections (one stacked product) -> per-head RMSNorm of q and k, not v
-> position encoding of q and k -> k, v written to the cache -> attention of every query
over its sequence's keys at positions <= its own (and inside the window, if the layer has
one) -> output projection.  The result is returned as a delta for the residual stream.

Sizes and constants (heads, groups, head size, biases, q/k norm and its eps, window, scale)
are parameters; a layer that reads another layer's cache projects only q.  Further parameters:
value heads of another size than the key heads (``v_head_dim``), a mask by blocks of positions
instead of a window (``chunk``), a sigmoid gate per head on the attention's result, read from the
layer's input (``gated``; "per_value": a gate for every value of every head), and, through the
position encoding, rotation by neighbouring pairs.  Beside a window, the first ``keep_first`` positions
may stay visible to every later query; the softmax's denominator may have one more term exp(``sink``)
that brings no value; queries and keys may be divided by their root mean square after the position
encoding (``qk_unit_norm``); biases may be given for some of the projections only; and the values that
a layer caches may be blended with those of an earlier layer of the same step (``value_mix``).
Three more parameters form one path of their own (``_forward_wide``): ``qk_norm`` "whole" (queries and keys are each
normalised over ALL their heads together, with a weight vector of that width, before the position encoding),
``head_temperature`` (query head n's scores are multiplied by a number of the layer, folded into the query) and
``talking_heads`` (after the softmax the heads' weights are mixed by a matrix of the layer, a'_n = sum_g M[n, g] a_g,
and head n applies a'_n to the values of its own key/value head).
Heads of unequal or odd sizes are written into the cache padded with zeros to one width that the
attention kernels take: zeros in queries and keys change no score, zeros in values give zeros
that are dropped before the output projection.
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
from .base import BuildEnv, DeferredNorm, Mixer, build_position, register_mixer
from .linear import Linear

# From this many tokens in a step the q | k | v projection normalises, rotates and caches in its own
# epilogue.  With fewer tokens a block has too few tiles to hide that epilogue behind the next tile's
# main loop, and the rotation kernel after a plain product is as fast or faster (measured at 1,024 and
# 2,048 tokens against 4,096).
PROMPT_FUSED_MIN_TOKENS = 4096

# Tensor-name stems by role, unless the spec's ``names`` says otherwise (the defaults are those of
# Hugging Face's Qwen3 checkpoints: rocml/src/weights/layer.rs:47-58 lists the same tensors under GGUF names).
TENSOR_NAMES = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj", "q_norm": "q_norm", "k_norm": "k_norm",
                "gate": "gate_proj", "value_mix": "value_mix", "talk": "head_mix", "temperature": "head_temperature"}

VALUE_MIX_SOURCE = "attention.value_mix_source"    # where a step keeps the source layer's values (StepBatch.scratch)

DECODE_CHUNK = 64   # keys per split of decode attention (one page); fixed, so a row's sums never depend on the batch


@register_mixer("attention")
class Attention(Mixer):
    graph_safe = True

    def __init__(self, spec: MixerSpec, hidden: int, env: BuildEnv):
        p = spec.params
        self.env = env
        self.hidden = hidden
        self.nq = int(p["n_heads"])
        self.nkv = int(p["n_kv_heads"])
        self.hd = int(p["head_dim"])
        if self.nq <= 0 or self.nkv <= 0 or self.nq % self.nkv:
            raise ConfigError(f"{self.nq} query heads cannot be grouped over {self.nkv} key/value heads")
        self.vd = int(p.get("v_head_dim") or self.hd)
        self.gated = bool(p.get("gated", False))
        self.gate_per_value = p.get("gated") == "per_value"
        self.hdp = -(-max(self.hd, self.vd) // 16) * 16         # the width of every head in the cache
        if min(self.hd, self.vd) <= 0 or self.hdp > 512:
            raise ConfigError(f"head sizes {self.hd} (keys) and {self.vd} (values) are not supported: 1 to 512")
        bias = p.get("bias", False)
        self.bias = bool(bias)
        self.qk_norm = bool(p.get("qk_norm", False))
        self.qk_norm_whole = p.get("qk_norm") == "whole"
        self.head_temperature = bool(p.get("head_temperature", False))
        self.talking_heads = bool(p.get("talking_heads", False))
        self.wide = self.qk_norm_whole or self.head_temperature or self.talking_heads
        self.qk_norm_eps = float(p.get("qk_norm_eps", 1e-6))
        self.qk_unit_norm = bool(p.get("qk_unit_norm", False))
        self.window = p.get("window")
        self.chunk = p.get("chunk")
        self.keep_first = int(p.get("keep_first") or 0) if self.window else 0
        self.sink = None if p.get("sink") is None else float(p["sink"])
        self.value_mix = p.get("value_mix")
        if self.value_mix not in (None, "source", "mix"):
            raise ConfigError(f"attention: value_mix is 'source' or 'mix', found {self.value_mix!r}")
        if self.keep_first < 0:
            raise ConfigError("attention: keep_first counts positions and cannot be negative")
        if self.window and self.chunk:
            raise ConfigError("attention: a layer has a window or blocks of positions, not both")
        if self.wide and (self.gated or self.keep_first or self.sink is not None or self.qk_unit_norm or self.value_mix or
                          (self.qk_norm and not self.qk_norm_whole) or p.get("shares_cache")):
            raise ConfigError("attention: a norm over whole projections, head temperatures and mixed heads do not combine with "
                              "gates, kept first keys, a sink, unit norms, blended values, per-head norms or a shared cache")
        if self.talking_heads and self.nkv * self.nq * self.hdp > 65535 * 16:
            raise ConfigError("attention: too many heads to mix")
        if (self.window is not None and int(self.window) < 1) or (self.chunk is not None and int(self.chunk) < 1):
            raise ConfigError("attention: a window or a block of positions holds at least one position")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.hd)
        self.shares_cache = bool(p.get("shares_cache", False))  # set by the model for a reading layer
        self.position = build_position(spec.position, self.hd, env)
        # the plain layout: equal head sizes that the kernels take as they are, rotate-half pairs, no gate
        self.plain = not self.wide and self.vd == self.hd == self.hdp and not self.gated and \
            not (self.position.inv_freq is not None and getattr(self.position, "interleaved", False)) and \
            not (self.keep_first or self.sink is not None or self.qk_unit_norm or self.value_mix)
        if not self.plain and self.shares_cache:
            raise ConfigError("attention: a layer that reads another layer's cache must have the plain layout")
        qd, kvd = self.nq * self.hd, self.nkv * self.hd
        try:
            self.names = n = tensor_names(p, TENSOR_NAMES)
        except ValueError as e:
            raise ConfigError(f"attention: {e}") from None
        if not isinstance(bias, bool):          # the roles that have a bias, by name
            unknown = sorted(set(bias) - {"q", "k", "v", "o", "gate"})
            if unknown:
                raise ConfigError(f"attention: biases for unknown projections {unknown}")
            in_bias, o_bias = [n[r] for r in bias if r != "o"], "o" in bias
        else:
            in_bias, o_bias = bias, bias
        if self.shares_cache:
            self.qkv = Linear([n["q"]], [qd], hidden, in_bias, env)
        else:
            stems, outs = [n["q"], n["k"], n["v"]], [qd, kvd, self.nkv * self.vd]
            if self.gated:
                stems, outs = stems + [n["gate"]], outs + [self.nq * self.vd if self.gate_per_value else self.nq]
            self.qkv = Linear(stems, outs, hidden, in_bias, env)
        self.o = Linear([n["o"]], [hidden], self.nq * self.vd, o_bias, env)
        self.q_norm_w: Optional[torch.Tensor] = None
        self.k_norm_w: Optional[torch.Tensor] = None
        self.v_lambda: Optional[torch.Tensor] = None     # float32 [1] on the device: the share of the source layer's values
        self.talk: Optional[torch.Tensor] = None         # float32 [nq, nq]: the matrix that mixes the heads' weights
        self.temperature: Optional[torch.Tensor] = None  # float32 [nq]: a factor on every head's scores

    def cache_requirement(self):
        return KVRequirement(self.nkv, self.hdp, self.window, chunk=self.chunk, keep_first=self.keep_first)

    def _span(self) -> int:
        """The mask as the kernels take it: 0 every earlier key, n the last n keys, -n blocks of n positions."""
        if self.window:
            return int(self.window)
        return -int(self.chunk) if self.chunk else 0

    def declare(self, prefix: str) -> List[TensorDecl]:
        out = self.qkv.declare(prefix) + self.o.declare(prefix)
        if self.qk_norm_whole:
            out.append(TensorDecl(f"{prefix}{self.names['q_norm']}.weight", (self.nq * self.hd,), "norm"))
            out.append(TensorDecl(f"{prefix}{self.names['k_norm']}.weight", (self.nkv * self.hd,), "norm"))
        elif self.qk_norm:
            out.append(TensorDecl(f"{prefix}{self.names['q_norm']}.weight", (self.hd,), "norm"))
            if not self.shares_cache:
                out.append(TensorDecl(f"{prefix}{self.names['k_norm']}.weight", (self.hd,), "norm"))
        if self.talking_heads:
            out.append(TensorDecl(f"{prefix}{self.names['talk']}.weight", (self.nq, self.nq), "mixing"))
        if self.head_temperature:
            out.append(TensorDecl(f"{prefix}{self.names['temperature']}.weight", (self.nq,), "norm"))
        if self.value_mix == "mix":
            out.append(TensorDecl(f"{prefix}{self.names['value_mix']}.weight", (), "fraction"))
        return out

    def ignorable(self, prefix: str) -> List[str]:
        """A layer that does not blend its values may still carry the blend's number in the files."""
        return [] if self.value_mix == "mix" else [f"{prefix}{self.names['value_mix']}.weight"]

    def load(self, tensors: Dict[str, torch.Tensor], prefix: str) -> None:
        self.qkv.load(tensors, prefix)
        if not self.plain:
            self.qkv.pad_rows(8)     # a stack with a few gate rows is rarely a multiple of 8 wide
        self.o.load(tensors, prefix)
        if self.talking_heads:
            self.talk = tensors[f"{prefix}{self.names['talk']}.weight"].float().contiguous()
        if self.head_temperature:
            self.temperature = tensors[f"{prefix}{self.names['temperature']}.weight"].float().contiguous()
        if self.qk_norm_whole:         # 32-bit vectors, as the kernel of this path reads them
            self.q_norm_w = tensors[f"{prefix}{self.names['q_norm']}.weight"].float().contiguous()
            self.k_norm_w = tensors[f"{prefix}{self.names['k_norm']}.weight"].float().contiguous()
        elif self.qk_norm:
            self.q_norm_w = tensors[f"{prefix}{self.names['q_norm']}.weight"]
            self.k_norm_w = self.q_norm_w if self.shares_cache else tensors[f"{prefix}{self.names['k_norm']}.weight"]
            if self.k_norm_w.dtype != self.q_norm_w.dtype:
                self.q_norm_w, self.k_norm_w = self.q_norm_w.float(), self.k_norm_w.float()
        if self.value_mix == "mix":
            self.v_lambda = tensors[f"{prefix}{self.names['value_mix']}.weight"].float().reshape(1).contiguous()

    def weight_bytes(self) -> int:
        return self.qkv.weight_bytes() + self.o.weight_bytes()

    def workspace_bytes(self, n_tokens: int) -> int:
        """Projections, attention output and the delta (as partial sums: up to 8 of each for few tokens)."""
        esz = 4 if self.env.mode == "float32" else 2
        parts = 8 if n_tokens <= 128 else 1
        return n_tokens * (self.qkv.n * max(esz, 4 * parts if parts > 1 else esz) + 3 * self.nq * self.hdp * esz
                           + self.hidden * 4 * parts + self.nq * 4 * (self.hdp + 2) * (parts if parts > 1 else 0))

    def cost(self, q_lens, kv_lens):
        from ..profile import cost as C
        T = sum(q_lens)
        esz = 4 if self.env.mode == "float32" else 2
        parts = [self.qkv.cost(T), self.o.cost(T),
                 C.attention(q_lens, kv_lens, self.nq, self.nkv, self.hdp, esz, self._span() or None)]
        return sum(p[0] for p in parts), sum(p[1] for p in parts)

    can_sink = True        # forward() accepts sink=ResidualSink (see parts.base)

    def takes_deferred(self, batch) -> bool:
        """Whether forward() can be handed a DeferredNorm for this step: the decode kernel that takes
        the projections applies the rows' 1/RMS, which a bias inside the projection would spoil."""
        return (batch.is_decode and self.plain and self.hd == 128 and not self.bias and self.env.act_dtype == torch.bfloat16
                and self.qkv.weight is not None and self.qkv.weight.dtype == torch.bfloat16
                and self.qkv._splits(batch.n_tokens) > 1
                and (self.shares_cache or self.nq // self.nkv <= 16)     # wider groups: the kernel does not write the cache
                and (self.position.inv_freq is None or self.position.rot_dim == self.hd))

    can_add_into = True    # forward() accepts add_into=residual (see parts.base)

    def forward(self, xn, batch, view, sink=None, add_into=None):
        T = batch.n_tokens
        dev, act = self.env.device, self.env.act_dtype
        qd = self.nq * self.hd
        window = self._span()
        writes = view.writes and not self.shares_cache
        if self.wide:
            return self._forward_wide(xn, batch, view, window, sink, add_into)
        if not self.plain:
            return self._forward_padded(xn, batch, view, window, writes, sink, add_into)
        attn = torch.empty((T, qd), dtype=act, device=dev)
        done = False
        if isinstance(xn, DeferredNorm):
            proj = self.qkv.forward_auto(xn.x, T)
            done = self._decode_fused(proj, attn, batch, view, window, writes, xn.rowscale, xn.width)
            if not done:
                xn = xn.materialize()     # the kernel declined after all: the norm's own kernel, then as always
        if not done and not batch.is_decode and self._prompt_fused(xn, attn, batch, view, window, writes):
            done = True
        if not done:
            proj = self.qkv.forward_auto(xn, T)      # [T, N] or [S, T, N] partial sums
            done = batch.is_decode and self._decode_fused(proj, attn, batch, view, window, writes)
        if not done:
            q = proj if proj.dim() == 2 else torch.empty((T, qd), dtype=act, device=dev)
            kernels.qk_norm_rope_cache(
                proj, q, T, self.nq, self.nkv, self.hd, self.q_norm_w, self.k_norm_w, self.qk_norm_eps,
                self.position.inv_freq, self.position.rot_dim, batch.positions, batch.slot_of_token,
                view.block_table, view.k, view.v, write_kv=writes,
                cos_sin=self.position.cos_sin(batch))
            self.attend(q, attn, batch, view, window)
        if sink is not None:
            deferred = self.o.forward_residual(attn, T, sink)
            if deferred is not None:
                return deferred
        if add_into is not None and self.o.forward_add(attn, T, add_into):
            return None
        return self.o.forward_delta(attn, T)

    def _forward_padded(self, xn, batch, view, window, writes, sink, add_into):
        """Heads of unequal sizes, neighbouring rotation pairs or a gate per head: one kernel rotates and pads
        queries and keys, writes keys and values (padded) to their pages and takes the sigmoid of the gate
        columns; the attention runs at the padded head size; one kernel multiplies each head by its gate and
        drops the padding."""
        T = batch.n_tokens
        dev, act = self.env.device, self.env.act_dtype
        if isinstance(xn, DeferredNorm):
            xn = xn.materialize()
        proj = self.qkv.forward_auto(xn, T)
        # values blended across layers: the source layer leaves its own for the step's later layers
        v_out = v_first = None
        if self.value_mix == "source":
            v_out = batch.scratch[VALUE_MIX_SOURCE] = torch.empty((T, self.nkv * self.vd), dtype=torch.float32, device=dev)
        elif self.value_mix == "mix":
            v_first = batch.scratch.get(VALUE_MIX_SOURCE)
            if v_first is None or v_first.shape != (T, self.nkv * self.vd):
                raise ConfigError("attention: a layer blends its values with a source layer's, which must run before it "
                                  "in the same step with the same key/value heads and value size")
        # a raw gate for every value of heads that carry no padding: an attention kernel that takes the projection's gate
        # columns multiplies its result by their sigmoid as it writes it
        raw_gate = None
        if self.gate_per_value and self.hdp == self.vd:
            off = self.nq * self.hd + self.nkv * (self.hd + self.vd)
            raw_gate = proj[..., off:off + self.nq * self.vd]
        # one token a sequence, heads of 128 on both sides: the attention kernel makes the heads from the projection's
        # partial sums itself (norm, partial rotation, division by the root mean square, blended values, the cache write)
        if batch.is_decode and writes and self.hd == self.vd == self.hdp and (raw_gate is not None or not self.gated):
            attn = torch.empty((T, self.nq * self.hd), dtype=act, device=dev)
            if self._decode_fused(proj, attn, batch, view, window, writes, v_first=v_first, v_keep=v_out, gate=raw_gate):
                return self._project_out(attn, T, sink, add_into)
        q = torch.empty((T, self.nq * self.hdp), dtype=act, device=dev)
        gates = torch.empty((T, self.nq), dtype=torch.float32, device=dev) if self.gated and not self.gate_per_value else None
        with scope(op="rotate_cache"):
            kernels.qk_norm_rope_cache(
                proj, q, T, self.nq, self.nkv, self.hd, self.q_norm_w, self.k_norm_w, self.qk_norm_eps,
                self.position.inv_freq, self.position.rot_dim, batch.positions, batch.slot_of_token,
                view.block_table, view.k, view.v, write_kv=writes, cos_sin=self.position.cos_sin(batch),
                v_head_dim=self.vd, padded_head_dim=self.hdp, interleaved=getattr(self.position, "interleaved", False),
                gates=gates, post_norm=self.qk_unit_norm, v_first=v_first, v_lambda=self.v_lambda if v_first is not None else None,
                v_out=v_out)
        attn = torch.empty((T, self.nq * self.hdp), dtype=act, device=dev)
        gated_inside = paged_attention(q, attn, batch, view.k, view.v, view.block_table, self.nq, self.nkv, self.hdp, self.scale,
                                       window, keep=self.keep_first, sink=self.sink, gate=raw_gate)
        if (self.gated and not gated_inside) or self.hdp != self.vd:
            narrow = torch.empty((T, self.nq * self.vd), dtype=act, device=dev)
            raw = None
            if self.gate_per_value:          # the gate's columns of the projection rows, as they are: the kernel takes the sigmoid
                off = self.nq * self.hd + self.nkv * (self.hd + self.vd)
                raw = proj[..., off:off + self.nq * self.vd]
            with scope(op="head_gate"):
                kernels.head_gate(attn, narrow, gates, self.nq, self.hdp, self.vd, T, raw=raw, per_value=self.gate_per_value)
            attn = narrow
        return self._project_out(attn, T, sink, add_into)

    def _forward_wide(self, xn, batch, view, window, sink, add_into):
        """A norm over the whole q and k projections, a temperature per head, the heads' weights mixed after the softmax.

        One kernel normalises, rotates, scales and pads the queries and writes keys and values to their pages.  Mixing
        weights and then applying them to values is the same as applying every head's own weights to the values of every
        stored head and then mixing the results: o_n = sum_g M[n, g] (a_g . V_m(n)).  So the attention runs once over
        (key head, value head) pairs (``cross``), and a small kernel forms the sums over g in 32-bit."""
        T = batch.n_tokens
        dev, act = self.env.device, self.env.act_dtype
        if isinstance(xn, DeferredNorm):
            xn = xn.materialize()
        proj = self.qkv.forward_auto(xn, T)
        rot = self.position.rot_dim if self.position.inv_freq is not None else 0
        q = torch.empty((T, self.nq * self.hdp), dtype=act, device=dev)
        with scope(op="rotate_cache"):
            kernels.wide_norm_rope_cache(proj, q, T, self.nq, self.nkv, self.hd, self.vd, self.hdp, self.q_norm_w, self.k_norm_w,
                                         self.qk_norm_eps, self.temperature, self.position.cos_sin(batch) if rot else None, rot,
                                         getattr(self.position, "interleaved", False), batch.positions, batch.slot_of_token,
                                         view.block_table, view.k, view.v)
        pairs = self.nkv if self.talking_heads and self.nkv > 1 else 1
        wide = torch.empty((T, self.nq * pairs * self.hdp), dtype=act, device=dev)
        paged_attention(q, wide, batch, view.k, view.v, view.block_table, self.nq * pairs, self.nkv * pairs, self.hdp, self.scale,
                        window, cross=pairs if pairs > 1 else 0)
        if self.talking_heads:
            attn = torch.empty((T, self.nq * self.vd), dtype=act, device=dev)
            with scope(op="mix_heads"):
                kernels.talk_mix(wide, self.talk, attn, self.nq, self.nkv, self.hdp, self.vd, batch.slot_of_token, T)
        elif self.hdp != self.vd:
            attn = torch.empty((T, self.nq * self.vd), dtype=act, device=dev)
            with scope(op="head_gate"):
                kernels.head_gate(wide, attn, None, self.nq, self.hdp, self.vd, T)
        else:
            attn = wide
        return self._project_out(attn, T, sink, add_into)

    def _project_out(self, attn, T, sink, add_into):
        if sink is not None:
            deferred = self.o.forward_residual(attn, T, sink)
            if deferred is not None:
                return deferred
        if add_into is not None and self.o.forward_add(attn, T, add_into):
            return None
        return self.o.forward_delta(attn, T)

    def _prompt_fused(self, xn, out, batch, view, window, writes) -> bool:
        """Many tokens, head size 128: the projection's own epilogue normalises and rotates the heads
        and writes keys and values into the cache, so the projections never go through memory.
        False: not this time (other sizes, a partial rotation, few tokens)."""
        if self.hd != 128 or self.env.act_dtype != torch.bfloat16 or not isinstance(xn, torch.Tensor) \
                or xn.dtype != torch.bfloat16 or self.qkv.weight is None or self.qkv.weight.dtype != torch.bfloat16:
            return False
        rot = self.position.rot_dim if self.position.inv_freq is not None else 0
        if rot not in (0, self.hd) or writes != (self.qkv.n == (self.nq + 2 * self.nkv) * self.hd):
            return False
        T = batch.n_tokens
        if T < PROMPT_FUSED_MIN_TOKENS:
            return False
        q = torch.empty((T, self.nq * self.hd), dtype=torch.bfloat16, device=xn.device)
        cos_sin = self.position.cos_sin(batch) if rot else None
        with scope(op=self.qkv.label):
            if not kernels.gemm_tcgen05_qkv_rope(
                    xn, self.qkv.weight, q, self.nq, self.nkv, self.q_norm_w, self.k_norm_w, self.qk_norm_eps,
                    cos_sin, batch.positions, batch.slot_of_token,
                    view.block_table, view.k, view.v, self.qkv.bias, T):
                return False
        self.attend(q, out, batch, view, window)
        return True

    def _decode_fused(self, proj, out, batch, view, window, writes, rowscale=None, row_width=0, v_first=None, v_keep=None,
                      gate=None) -> bool:
        """One token per sequence, head size 128, float32 projections: the attention kernel itself
        adds the partial sums, normalises and rotates the queries and writes the new key and value,
        so no kernel stands between the projection and the attention.  False: not this time."""
        if self.hd != 128 or proj.dtype != torch.float32 or view.k.dtype != torch.bfloat16:
            return False
        rot = self.position.rot_dim if self.position.inv_freq is not None else 0
        if rot % 8 or getattr(self.position, "interleaved", False) or (writes and self.nq // self.nkv > 16):
            return False
        n_pages = max(1, (batch.max_kv_len + DECODE_CHUNK - 1) // DECODE_CHUNK)
        groups = self.nkv * ((self.nq // self.nkv + 15) // 16)
        n_blocks, ppb = kernels.decode_split(batch.n_seqs, groups, n_pages, out.device)
        if self.keep_first and ppb == 0:         # kept first keys: a sequence takes whole blocks (see paged_attention)
            ppb = -(-n_pages // min(n_pages, kernels.DECODE_CLUSTER_MAX))
            n_blocks = -(-n_pages // ppb)
        acc = ml = None
        if n_pages > 1:
            T = batch.n_tokens
            parts = max(n_pages, n_blocks)          # the kernel strides a row's partial results by n_blocks
            acc = torch.empty((T, self.nq, parts, self.hd), dtype=torch.float32, device=out.device)
            ml = torch.empty((T, self.nq, parts, 2), dtype=torch.float32, device=out.device)
        return kernels.attention_decode_fused(
            proj, out, view.k, view.v, view.block_table, batch.seq_slot, batch.cu_q, batch.kv_len, batch.n_seqs,
            self.nq, self.nkv, self.hd, self.q_norm_w, self.k_norm_w, self.qk_norm_eps,
            self.position.cos_sin(batch) if rot else None, writes, self.scale, window, n_blocks, acc, ml, ppb,
            rowscale=rowscale, row_width=row_width, keep=self.keep_first, sink=self.sink, rot_dim=rot,
            post_norm=self.qk_unit_norm, v_first=v_first, v_lambda=self.v_lambda if v_first is not None else None,
            v_keep=v_keep, gate=gate)

    def attend(self, q, out, batch, view, window):
        """Softmax attention of the step's queries over the cache (see ``paged_attention``)."""
        paged_attention(q, out, batch, view.k, view.v, view.block_table, self.nq, self.nkv, self.hd, self.scale, window)


def paged_attention(q, out, batch, k_cache, v_cache, block_table, nq, nkv, hd, scale, window, keep=0, sink=None, gate=None,
                    cross=0) -> bool:
    """Softmax attention of the step's queries (rows of nq heads of ``hd``) over paged keys and values
    [pages, nkv, 64, hd], causal, inside ``window`` when it is not 0 (and the first ``keep`` positions beside it);
    ``sink``: a score whose exponential joins every row's denominator.  One token per sequence:
    keys split in fixed chunks, partial results merged; otherwise whole rows.  Any mixer whose cache is
    such pages calls this (keys and values may be the same tensor).  ``gate``: nq * hd columns of the step's projection
    rows ([T, ..] or partial sums [S, T, ..]); a kernel that takes them multiplies its result by their sigmoid.
    Returns whether that was done: if not, the result is as without ``gate`` and the caller gates it.
    ``cross`` (n > 1, the cache's own number of key/value heads): every query head's weights are applied to the values of
    every stored head; nkv = n * n then counts (key head, value head) pairs and nq = n * query heads the results."""
    if batch.is_decode:
        chunk = DECODE_CHUNK
        T = batch.n_tokens
        n_pages = max(1, (batch.max_kv_len + chunk - 1) // chunk)
        groups = nkv * ((nq // nkv + 15) // 16)
        n_blocks, ppb = kernels.decode_split(batch.n_seqs, groups, n_pages, q.device)
        if keep and ppb == 0:
            # equal shares of all sequences' pages count a sequence's pages from its window's first; with kept
            # first keys a sequence takes whole blocks instead
            ppb = -(-n_pages // min(n_pages, kernels.DECODE_CLUSTER_MAX))
            n_blocks = -(-n_pages // ppb)
        acc = ml = None
        if n_pages > 1:
            parts = max(n_pages, n_blocks)
            acc = torch.empty((T, nq, parts, hd), dtype=torch.float32, device=q.device)
            ml = torch.empty((T, nq, parts, 2), dtype=torch.float32, device=q.device)
        fast = kernels.attention_decode(q, out, k_cache, v_cache, block_table, batch.seq_slot, batch.cu_q,
                                        batch.kv_len, batch.n_seqs, nq, nkv, hd, scale,
                                        window, n_blocks, acc, ml, ppb, keep=keep, sink=sink, gate=gate, cross=cross)
        n_chunks = n_pages
        if fast:
            return gate is not None
        if n_chunks > 1:
            kernels.attention_generic(q, out, k_cache, v_cache, block_table, batch.seq_slot, batch.cu_q,
                                      batch.kv_len, batch.n_seqs, 1, nq, nkv, hd, scale,
                                      window, chunk, n_chunks, acc, ml, keep=keep, sink=sink, cross=cross)
            kernels.attention_merge(acc, ml, out, batch.positions, batch.slot_of_token, T, nq, hd,
                                    chunk, n_chunks, window, keep=keep, sink=sink)
            return False
    tc5_gate = gate if gate is not None and gate.dim() == 2 and gate.dtype == torch.bfloat16 else None
    if kernels.attention_prefill_tc5(q, batch.n_tokens, out, k_cache, v_cache, block_table, batch.seq_slot,
                                     batch.cu_q, batch.kv_len, batch.n_seqs, batch.max_q_len, nq, nkv,
                                     hd, scale, window, max_kv_len=batch.max_kv_len, keep=keep, sink=sink, gate=tc5_gate, cross=cross):
        return tc5_gate is not None
    if cross <= 1 and kernels.attention_prefill(q, out, k_cache, v_cache, block_table, batch.seq_slot, batch.cu_q,
                                 batch.kv_len, batch.n_seqs, batch.max_q_len, nq, nkv, hd,
                                 scale, window, keep=keep, sink=sink):
        return False
    kernels.attention_generic(q, out, k_cache, v_cache, block_table, batch.seq_slot, batch.cu_q,
                              batch.kv_len, batch.n_seqs, batch.max_q_len, nq, nkv, hd,
                              scale, window, keep=keep, sink=sink, cross=cross)
    return False

