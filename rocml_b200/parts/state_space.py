"""A state-space mixer with a step size per token and head (the dual form of a selective scan).

    [z | x | B | C | r] = Win h            z, x: heads * head_dim;  B, C: groups * state;  r: heads
    x, B, C <- silu(causal convolution over the last `conv_taps` tokens, per channel, with bias)
    dt = softplus(r + dt_bias)             per head
    S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T      per head, S [state, head_dim], zero when the sequence starts;
                                                          head n reads B and C of group n // (heads / groups)
    y_t = S_t^T C_t + D x_t
    out = Wo (norm_parts(y * silu(z)) * w)  the gated rows divided by their root mean square in `norm_groups` equal parts

What a sequence keeps, whatever its length: the state (``StateRequirement`` [heads, state, head_dim], 32-bit) and the
convolution's last conv_taps - 1 inputs (a second state, [conv_taps - 1, channels]).  One stacked product makes the
five blocks of columns from the layer's input; one kernel convolves and applies silu (32-bit out); one kernel carries the
step's tokens through the recurrence from the state the step before left (single tokens and short pieces token after
token; prompts by blocks of 64 tokens that run side by side, four kernels; one token a sequence with the state streaming
through registers); one kernel gates and normalises; the output
product is the one every mixer uses.  From the projection on everything is 32-bit: step sizes, decays, state, sums,
the gate, the norm.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from ..cache.requirements import BundleRequirement, StateRequirement
from ..config.specs import MixerSpec, tensor_names
from ..errors import ConfigError
from ..profile import scope
from ..weights.decl import TensorDecl
from .base import BuildEnv, DeferredNorm, Mixer, register_mixer
from .linear import Linear

# A step whose longest sequence brings more tokens than this runs the recurrence by blocks of 64 tokens side by side
# (three kernels); up to it, token after token in one kernel (also every decode step).
BLOCKS_MIN_TOKENS = 16

TENSOR_NAMES = {"in": "in_proj", "conv": "conv", "dt_bias": "dt_bias", "a_log": "A_log", "skip": "D", "norm": "norm", "o": "out_proj"}


@register_mixer("state_space")
class StateSpace(Mixer):
    graph_safe = True

    def __init__(self, spec: MixerSpec, hidden: int, env: BuildEnv):
        p = spec.params
        self.env = env
        self.hidden = hidden
        self.heads = int(p["n_heads"])
        self.hd = int(p["head_dim"])
        self.n = int(p["state"])
        self.groups = int(p.get("groups", 1))
        self.taps = int(p.get("conv_taps", 1))
        self.norm_groups = int(p.get("norm_groups", 1))
        self.norm_eps = float(p.get("norm_eps", 1e-6))
        if min(self.heads, self.hd, self.n, self.groups, self.taps, self.norm_groups) <= 0:
            raise ConfigError("state_space: heads, sizes, groups and taps must be positive")
        if self.heads % self.groups:
            raise ConfigError(f"state_space: {self.heads} heads cannot share {self.groups} groups of B and C")
        self.inner = self.heads * self.hd
        if self.inner % self.norm_groups:
            raise ConfigError(f"state_space: the {self.inner} gated values do not split in {self.norm_groups} equal parts")
        if self.taps > kernels.CONV_MAX_TAPS:
            raise ConfigError(f"state_space: a convolution of {self.taps} taps is not built (at most {kernels.CONV_MAX_TAPS})")
        if spec.position.kind != "none":
            raise ConfigError("state_space: a position encoding inside the mixer is not part of it")
        try:
            self.names = n = tensor_names(p, TENSOR_NAMES)
        except ValueError as e:
            raise ConfigError(f"state_space: {e}") from None
        gn = self.groups * self.n
        self.channels = self.inner + 2 * gn                 # what the convolution sees: x | B | C
        # columns of the projection: z | x | B | C | r
        self.z_off, self.conv_off, self.dt_off = 0, self.inner, 2 * self.inner + 2 * gn
        self.proj = Linear([n["in"]], [2 * self.inner + 2 * gn + self.heads], hidden, False, env)
        self.o = Linear([n["o"]], [hidden], self.inner, False, env)
        self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.skip = self.norm_w = None

    def cache_requirement(self):
        main = StateRequirement((self.heads, self.n, self.hd), torch.float32)
        if self.taps == 1:
            return main
        return BundleRequirement.of(main, conv=StateRequirement((self.taps - 1, self.channels), torch.float32))

    def _small(self, prefix: str):
        n = self.names
        return [("conv_w", f"{prefix}{n['conv']}.weight", (self.channels, self.taps), "matrix"),
                ("conv_b", f"{prefix}{n['conv']}.bias", (self.channels,), "bias"),
                ("dt_bias", f"{prefix}{n['dt_bias']}.weight", (self.heads,), "norm"),
                ("a_log", f"{prefix}{n['a_log']}.weight", (self.heads,), "norm"),
                ("skip", f"{prefix}{n['skip']}.weight", (self.heads,), "norm"),
                ("norm_w", f"{prefix}{n['norm']}.weight", (self.inner,), "norm")]

    def declare(self, prefix: str) -> List[TensorDecl]:
        return self.proj.declare(prefix) + self.o.declare(prefix) + [TensorDecl(name, shape, role)
                                                                     for _, name, shape, role in self._small(prefix)]

    def load(self, tensors: Dict[str, torch.Tensor], prefix: str) -> None:
        self.proj.load(tensors, prefix)
        self.proj.pad_rows(8)
        self.o.load(tensors, prefix)
        for attr, name, _, _ in self._small(prefix):
            setattr(self, attr, tensors[name].float().contiguous())        # 32-bit: they enter the recurrence

    def weight_bytes(self) -> int:
        return self.proj.weight_bytes() + self.o.weight_bytes() + 4 * (self.channels * (self.taps + 1) + 3 * self.heads + self.inner)

    def workspace_bytes(self, n_tokens: int) -> int:
        esz = 4 if self.env.mode == "float32" else 2
        parts = 8 if n_tokens <= 128 else 1
        blocks = (n_tokens // 64 + 8) * (self.heads * (self.n * self.hd + 1) + self.groups * 4096) * 4 if n_tokens > BLOCKS_MIN_TOKENS else 0
        return n_tokens * (self.proj.n * max(esz, 4 * parts if parts > 1 else esz) + self.channels * 4 + self.inner * (4 + esz)
                           + self.hidden * 4 * parts) + blocks

    def cost(self, q_lens, kv_lens):
        T = sum(q_lens)
        live = sum(1 for n in q_lens if n > 0)
        scan = (T * 4 * (self.channels + self.inner) + 8 * live * self.heads * self.n * self.hd, 6 * T * self.heads * self.n * self.hd)
        parts = [self.proj.cost(T), self.o.cost(T), scan]
        return sum(p[0] for p in parts), sum(p[1] for p in parts)

    def forward(self, xn, batch, view):
        T = batch.n_tokens
        dev, act = self.env.device, self.env.act_dtype
        if isinstance(xn, DeferredNorm):
            xn = xn.materialize()
        proj = self.proj.forward_auto(xn, T)          # [T, N] in the activations' type, or [S, T, N] float32 partial sums
        gn = self.groups * self.n
        u = torch.empty((T, self.channels), dtype=torch.float32, device=dev)
        with scope(op="causal_conv"):
            kept = view.extras["conv"].state if self.taps > 1 else None
            kernels.causal_conv(proj, T, self.conv_off, self.channels, self.taps, self.conv_w, self.conv_b, "silu", kept,
                                batch.seq_slot, batch.cu_q, batch.n_seqs, batch.max_q_len, u)
        y = torch.empty((T, self.inner), dtype=torch.float32, device=dev)
        with scope(op="ssm_scan"):
            if not batch.is_decode and batch.max_q_len > BLOCKS_MIN_TOKENS:
                blocks = T // kernels.SSM_BLOCK + batch.n_seqs
                work = torch.empty((blocks, self.heads, self.n, self.hd), dtype=torch.float32, device=dev)
                decay = torch.empty((blocks, self.heads), dtype=torch.float32, device=dev)
                cb = torch.empty((blocks, self.groups, kernels.SSM_BLOCK, kernels.SSM_BLOCK), dtype=torch.float32, device=dev)
                kernels.ssm_scan_blocks(u, T, 0, self.inner, self.inner + gn, proj, self.dt_off, self.dt_bias, self.a_log, self.skip,
                                        self.heads, self.groups, self.n, self.hd, view.state, batch.seq_slot, batch.cu_q,
                                        batch.n_seqs, y, work, decay, cb)
            else:
                kernels.ssm_scan(u, T, 0, self.inner, self.inner + gn, proj, self.dt_off, self.dt_bias, self.a_log, self.skip,
                                 self.heads, self.groups, self.n, self.hd, view.state, batch.seq_slot, batch.cu_q, batch.n_seqs, y,
                                 one_token_each=batch.is_decode)
        g = torch.empty((T, self.inner), dtype=act, device=dev)
        with scope(op="gate_norm"):
            kernels.gate_group_norm(y, proj, self.z_off, self.norm_w, self.norm_eps, self.norm_groups, "silu", g,
                                    batch.slot_of_token, T)
        return self.o.forward_delta(g, T)
