"""State-space mixer with a scalar decay per head (the Mamba-2 form of the state-space duality).

With ``inner = heads * head_dim``, N = ``state_dim`` and G = ``groups``, one input projection gives
``[z: inner | x: inner | B: G N | C: G N | dt: heads]``.  x, B and C pass a causal convolution per channel over
``taps`` tokens (with bias) and silu.  Per head h, which uses group ``h // (heads / G)``:

    dt' = softplus(dt + dt_bias[h]);   S <- exp(-exp(A_log[h]) dt') S + dt' B x^T;   y = S^T C + D[h] x

then ``y * silu(z)`` is RMS-normed in ``norm_groups`` equal parts (the gate comes before the norm), multiplied by a
weight, and projected back.  Per request the part keeps two fixed-size states in the slot pool, both float32 and zero
when the request starts: the convolution's last ``taps - 1`` inputs and S [heads, head_dim, N].  The step sizes, the
decay, S and the norm are float32; the projections and the convolution's output are in the compute dtype.
"""

from __future__ import annotations

import torch

from slipstream_b200 import ops

from .base import MIXERS, LayerBinding, Mixer, Runtime, StateSpec, WeightSpec


@MIXERS.register("state_space")
class StateSpaceMixer(Mixer):
    cuda_graph_safe = True

    def __init__(self, name: str, hidden_size: int, heads: int, head_dim: int, state_dim: int, groups: int = 1,
                 taps: int = 4, norm_groups: int = 1, norm_eps: float = 1e-6, names: dict[str, str] | None = None) -> None:
        """``names``: the checkpoint's tensor names by role (in, conv, conv_bias, dt_bias, a_log, d, norm, out)."""
        if heads < 1 or groups < 1 or heads % groups:
            raise ValueError(f"heads ({heads}) must be a multiple of groups ({groups})")
        if not 1 <= taps <= 8 or not 1 <= state_dim <= 256 or head_dim < 1:
            raise ValueError("taps must be 1..8, state_dim 1..256, head_dim positive")
        if (heads * head_dim) % norm_groups:
            raise ValueError("the inner width does not split into norm_groups equal parts")
        self.name = name
        self.hidden_size = hidden_size
        self.heads, self.head_dim, self.state_dim, self.groups = heads, head_dim, state_dim, groups
        self.taps, self.norm_groups, self.norm_eps = taps, norm_groups, float(norm_eps)
        self.inner = heads * head_dim
        self.channels = self.inner + 2 * groups * state_dim  # what the convolution runs over: x, B, C
        self.proj_width = 2 * self.inner + 2 * groups * state_dim + heads
        n = name
        self.names = {"in": f"{n}.in_proj.weight", "conv": f"{n}.conv1d.weight", "conv_bias": f"{n}.conv1d.bias",
                      "dt_bias": f"{n}.dt_bias", "a_log": f"{n}.A_log", "d": f"{n}.D", "norm": f"{n}.norm.weight",
                      "out": f"{n}.out_proj.weight"}
        self.names.update(names or {})

    def weight_specs(self) -> list[WeightSpec]:
        n, h = self.names, self.hidden_size
        return [WeightSpec(n["in"], (self.proj_width, h)),
                WeightSpec(n["conv"], (self.channels, self.taps), init=("normal", 0.3)),
                WeightSpec(n["conv_bias"], (self.channels,), kind="vector"),
                WeightSpec(n["dt_bias"], (self.heads,), kind="vector", init=("normal", 0.5)),
                WeightSpec(n["a_log"], (self.heads,), kind="vector", init=("normal", 0.5)),
                WeightSpec(n["d"], (self.heads,), kind="vector", init=("one_plus_normal", 0.1)),
                WeightSpec(n["norm"], (self.inner,), kind="vector", init=("one_plus_normal", 0.1)),
                WeightSpec(n["out"], (h, self.inner))]

    def state_specs(self) -> list[StateSpec]:
        return [StateSpec("conv", (self.taps - 1, self.channels)),
                StateSpec("ssm", (self.heads, self.head_dim, self.state_dim))]

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        n = self.names
        # rows of zeros behind the projection bring its width to a multiple of 8, so that every token's row starts on a
        # 16-byte boundary (the kernels behind it then take 16 bytes a load); nobody reads the columns they make
        w_in = weights[n["in"]]
        pad = -w_in.shape[0] % 8
        self.in_weight = torch.cat([w_in, w_in.new_zeros((pad, w_in.shape[1]))]).contiguous() if pad else w_in
        self.out_weight = weights[n["out"]]
        as_f32 = lambda t: t.to(torch.float32).contiguous()  # noqa: E731  (exact: the stored values are kept)
        self.conv_taps, self.conv_bias = as_f32(weights[n["conv"]]), as_f32(weights[n["conv_bias"]])
        self.dt_bias, self.a_log, self.d_skip = as_f32(weights[n["dt_bias"]]), as_f32(weights[n["a_log"]]), as_f32(weights[n["d"]])
        self.norm_weight = as_f32(weights[n["norm"]])

    def weight_bytes(self) -> int:
        return (self.in_weight.numel() + self.out_weight.numel()) * self.out_weight.element_size()

    def forward(self, x: torch.Tensor, ctx, layer: LayerBinding) -> torch.Tensor:
        proj = ops.linear(x, self.in_weight)
        xbc = ops.conv_silu(proj, self.inner, self.channels, self.conv_taps, self.conv_bias, layer.state["conv"], ctx)
        y = ops.ssm_scan(xbc, proj[:, self.inner + self.channels: self.proj_width], self.dt_bias, self.a_log, self.d_skip,
                         layer.state["ssm"], ctx, self.heads, self.groups, self.head_dim, self.state_dim)
        gated = ops.group_norm(y, self.norm_weight, self.norm_groups, self.norm_eps, self.runtime.dtype,
                               gate=proj[:, : self.inner])
        return ops.linear(gated, self.out_weight)
