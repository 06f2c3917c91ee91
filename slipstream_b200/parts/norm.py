"""RMSNorm, fused with the residual add that precedes it.

``y = weight * round(x * rsqrt(mean(x^2) + eps))`` with the statistics in
float32 (slipstream/models/layers/rmsnorm.py:28-34).  The residual stream is kept
in float32; the branch output that has not been added yet comes in as ``delta``.
"""

from __future__ import annotations

import torch

from slipstream_b200 import ops

from .base import NORMS, Norm, Runtime, WeightSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    cuda_graph_safe = True

    def __init__(self, name: str, size: int, eps: float, tensor: str | None = None) -> None:
        """``tensor``: the checkpoint's name of the weight vector (default ``<name>.weight``)."""
        self.name = name
        self.size = size
        self.eps = float(eps)
        self.tensor = tensor or f"{name}.weight"
        self.weight: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(self.tensor, (self.size,), kind="vector", init=("one_plus_normal", 0.1))]

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        self.weight = weights[self.tensor]

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def add_norm(self, residual: torch.Tensor, delta: torch.Tensor | None,
                 rows: torch.Tensor | None = None) -> torch.Tensor:
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, self.runtime.dtype, rows=rows)

    def add_norm_of_linear(self, residual: torch.Tensor, x: torch.Tensor, weight: torch.Tensor,
                           bias: torch.Tensor | None) -> torch.Tensor:
        return ops.linear_add_rmsnorm(x, weight, bias, residual, self.weight, self.eps, self.runtime.dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.add_norm(x, None)


@NORMS.register("group_rmsnorm")
class GroupRMSNorm(Norm):
    """RMS norm in ``groups`` equal consecutive parts of the vector, each divided by its own
    ``sqrt(mean(part^2) + eps)``, the whole times a weight; float32 arithmetic, the weight kept in float32.

    Two uses.  As a model's last norm: ``add_norm(stream, None, rows)``.  On a branch's OUTPUT, for blocks that add
    ``norm(branch(x))`` to the stream (`BranchNormBlock`): ``add_branch(stream, y)`` adds the normed output in place
    and hands back the new stream in the compute dtype, which is what the next branch reads."""

    cuda_graph_safe = True

    def __init__(self, name: str, size: int, eps: float, groups: int = 1, tensor: str | None = None) -> None:
        if groups < 1 or size % groups:
            raise ValueError(f"{size} features do not split into {groups} equal groups")
        self.name = name
        self.size = size
        self.eps = float(eps)
        self.groups = int(groups)
        self.tensor = tensor or f"{name}.weight"
        self.weight: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(self.tensor, (self.size,), kind="vector", init=("one_plus_normal", 0.1))]

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        self.weight = weights[self.tensor].to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def add_norm(self, residual: torch.Tensor, delta: torch.Tensor | None,
                 rows: torch.Tensor | None = None) -> torch.Tensor:
        if delta is not None:
            raise ValueError("a grouped norm of the stream takes no pending branch output")
        return ops.group_norm(residual, self.weight, self.groups, self.eps, self.runtime.dtype, rows=rows)

    def add_branch(self, residual: torch.Tensor, y: torch.Tensor, *, gate: torch.Tensor | None = None, terms: int = 1,
                   extra: torch.Tensor | None = None, term_rows: torch.Tensor | None = None,
                   want_out: bool = True) -> torch.Tensor | None:
        """``residual += norm(y)`` in place; returns the new stream as a branch reads it (the stream itself in
        float32, its rounding in bfloat16; None with ``want_out`` False).  ``terms`` / ``extra``: ``y`` is a sum that
        has not been formed yet (`ops.group_norm`)."""
        fp32 = self.runtime.dtype == torch.float32
        out = ops.group_norm(y, self.weight, self.groups, self.eps, self.runtime.dtype, residual=residual, gate=gate,
                             terms=terms, extra=extra, term_rows=term_rows, want_out=want_out and not fp32)
        return residual if fp32 and want_out else out

    def forward(self, x: torch.Tensor, gate: torch.Tensor | None = None) -> torch.Tensor:
        """``norm(x)`` (``x`` in the compute dtype or float32), or ``norm(x * silu(gate))``."""
        return ops.group_norm(x, self.weight, self.groups, self.eps, self.runtime.dtype, gate=gate)


@NORMS.register("stream_rounding")
class StreamRounding(Norm):
    """What a block that norms its branches' OUTPUTS applies first: nothing but the rounding of the float32 stream
    to the compute dtype.  It stands where other blocks have their first norm, so that the block in front, which
    writes the stream last, can hand the rounded stream over (`Block.first_norm`)."""

    cuda_graph_safe = True

    def add_norm(self, residual: torch.Tensor, delta: torch.Tensor | None,
                 rows: torch.Tensor | None = None) -> torch.Tensor:
        if delta is not None or rows is not None:
            raise ValueError("the rounding of the stream takes no pending output and no selection of rows")
        return ops.round_stream(residual, self.runtime.dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.add_norm(x, None)
