"""Position encodings.  A mixer's fused kernel rotates queries and keys by the angles
pos * inv_freq[i]; the encoding owns that table, so another encoding (a partial rotation,
another base, scaled frequencies) is another table, not another kernel."""
from __future__ import annotations

import math

import torch

from ..config.specs import PositionSpec
from ..errors import ConfigError
from .base import BuildEnv, PositionEncoding, register_position


@register_position("none")
class NoPosition(PositionEncoding):
    graph_safe = True

    def __init__(self, spec: PositionSpec, head_dim: int, env: BuildEnv):
        self.inv_freq = None
        self.rot_dim = 0

    def cos_sin(self, batch):
        return None


def stretch_long_waves(inv: torch.Tensor, factor: float, low: float, high: float, original: float) -> torch.Tensor:
    """Frequencies with the long wavelengths stretched, piecewise by wavelength L = 2 pi / f: unchanged where
    L < original / high; f / factor where L > original / low; between the two a blend,
    s = (original / L - low) / (high - low), (1 - s) f / factor + s f.  Double precision in and out."""
    if not (factor > 0 and high > low >= 0 and original > 0):
        raise ConfigError(f"frequency scaling needs factor > 0, high > low >= 0 and original > 0 "
                          f"(found factor {factor}, low {low}, high {high}, original {original})")
    wave = 2.0 * math.pi / inv
    s = (original / wave - low) / (high - low)
    blend = (1.0 - s) * inv / factor + s * inv
    out = torch.where(wave < original / high, inv, blend)
    if low > 0:
        out = torch.where(wave > original / low, inv / factor, out)
    return out


# Constants of the ramp form of frequency scaling.
RAMP_MIN_WIDTH = 0.001         # the least the ramp's width (hi - lo) counts as
MAGNITUDE_SLOPE = 0.1          # cosines and sines are multiplied by MAGNITUDE_SLOPE * ln(factor) + 1


def blend_along_ramp(inv: torch.Tensor, theta: float, factor: float, original: float, fast: float, slow: float):
    """Frequencies blended between f (the fast pairs) and f / factor (the slow ones) along a ramp over the pair
    index i.  With n = 2 * len(inv) rotated entries, the index at which a wave turns t times over ``original``
    positions is d(t) = n ln(original / (2 pi t)) / (2 ln theta); lo = max(floor(d(fast)), 0),
    hi = min(ceil(d(slow)), n - 1), r_i = clamp((i - lo) / max(hi - lo, RAMP_MIN_WIDTH), 0, 1) and
    f_i <- r_i f_i / factor + (1 - r_i) f_i.  Returns (frequencies, magnitude), magnitude =
    MAGNITUDE_SLOPE * ln(factor) + 1, the factor on every cosine and sine.  Double precision in and out."""
    if not (factor > 0 and original > 0 and fast > 0 and slow > 0 and theta > 0 and theta != 1.0):
        raise ConfigError(f"frequency scaling along a ramp needs positive factor, original, fast and slow and a base "
                          f"other than 1 (found factor {factor}, original {original}, fast {fast}, slow {slow}, base {theta})")
    n = 2 * inv.numel()

    def turns_at(t: float) -> float:
        return n * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(theta))
    lo = max(math.floor(turns_at(fast)), 0)
    hi = min(math.ceil(turns_at(slow)), n - 1)
    i = torch.arange(inv.numel(), dtype=torch.float64)
    r = torch.clamp((i - lo) / max(hi - lo, RAMP_MIN_WIDTH), 0.0, 1.0)
    return inv / factor * r + inv * (1.0 - r), MAGNITUDE_SLOPE * math.log(factor) + 1.0


@register_position("rope_neox")
class RotaryNeox(PositionEncoding):
    """Rotate-half rotary embedding: inv_freq[i] = theta^(-2i / rot_dim) for i < rot_dim / 2,
    pairs (i, i + rot_dim / 2) (rocml-kernels/kernels/rope.hip:18-33).  The exponent and the
    power are evaluated in double precision and rounded once to float32; the angle
    pos * inv_freq and its sine and cosine are 32-bit, in the kernel.  Parameter ``scaling``
    ({factor, low, high, original}) stretches the long wavelengths (``stretch_long_waves``);
    parameter ``ramp_scaling`` ({factor, original, fast, slow}) blends the frequencies along a ramp
    and gives the step's table of cosines and sines a common ``magnitude`` (``blend_along_ramp``)."""

    graph_safe = True
    interleaved = False        # which entries of a head form a pair: (i, i + rot_dim / 2)
    kind = "rope_neox"

    def __init__(self, spec: PositionSpec, head_dim: int, env: BuildEnv):
        rot = head_dim if spec.rot_dim is None else int(spec.rot_dim)
        if rot <= 0 or rot % 2 or rot > head_dim:
            raise ConfigError(f"rotary dimension {rot} must be even and at most the head size {head_dim}")
        if not spec.theta > 0:
            raise ConfigError(f"rotary base must be positive, found {spec.theta}")
        self.rot_dim = rot
        self.theta = float(spec.theta)
        i = torch.arange(rot // 2, dtype=torch.float64)
        inv = torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64), -2.0 * i / rot)
        sc = spec.params.get("scaling")
        self.scaling = None
        if sc:
            sc = dict(sc)
            self.scaling = tuple(float(sc[k]) for k in ("factor", "low", "high", "original"))
            inv = stretch_long_waves(inv, *self.scaling)
        self.magnitude = 1.0        # the factor on every cosine and sine; it lives in the step's table
        ramp = spec.params.get("ramp_scaling")
        self.ramp_scaling = None
        if ramp:
            if sc:
                raise ConfigError("a rotation takes one form of frequency scaling, not both")
            ramp = dict(ramp)
            self.ramp_scaling = tuple(float(ramp[k]) for k in ("factor", "original", "fast", "slow"))
            inv, self.magnitude = blend_along_ramp(inv, self.theta, *self.ramp_scaling)
        self.inv_freq = inv.to(torch.float32).to(env.device)

    def cos_sin(self, batch):
        """(cos, sin) of every token's angles for this step, computed once and shared by all the
        layers that use this encoding with the same table."""
        from .. import kernels
        key = ("rope", self.rot_dim, self.theta, self.scaling, self.ramp_scaling)      # layers with the same angles share the table
        if key not in batch.scratch:
            batch.scratch[key] = kernels.rope_table(batch.positions, self.inv_freq, batch.n_tokens, self.magnitude)
        return batch.scratch[key]


@register_position("rope_pairs")
class RotaryPairs(RotaryNeox):
    """The same rotation with neighbouring entries as pairs: (2i, 2i + 1) turn by pos * inv_freq[i],
    i < rot_dim / 2; the entries from rot_dim on pass unchanged.  Same table, same parameters."""

    interleaved = True
    kind = "rope_pairs"


@register_position("sinusoid")
class SinusoidPosition(PositionEncoding):
    """A position vector added to the embedding output (a model's ``input_position``), not a rotation inside
    a mixer: entry 2i is sin(pos * theta^(-2i / width)), entry 2i + 1 the cosine of the same angle.  The
    exponent and the power are evaluated in double precision and rounded once to float32; the angle and its
    sine and cosine are 32-bit, in the embedding kernel.  ``head_dim`` here is the model's width."""

    graph_safe = True

    def __init__(self, spec: PositionSpec, head_dim: int, env: BuildEnv):
        if not spec.theta > 0:
            raise ConfigError(f"the sinusoid's base must be positive, found {spec.theta}")
        self.width = head_dim
        self.theta = float(spec.theta)
        self.rot_dim = 0
        i = torch.arange((head_dim + 1) // 2, dtype=torch.float64)
        inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / head_dim)
        self.inv_freq = inv.to(torch.float32).to(env.device)

    def cos_sin(self, batch):
        return None
