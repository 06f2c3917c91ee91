"""Builder of the Sarudra decoder from ``SarudraConfig``: which parts stand in which layer, with which constants
and tensor names.

Per layer ``l<i>`` a `BranchNormBlock` (``x + norm1(mixer(x))``, ``x + norm2(ffn(x))``, grouped RMS norms on the
branches' outputs) around one of two mixers and one of two feed-forwards, or none:

* ``mamba2``: a `StateSpaceMixer` (tensors ``l<i>.mix.{in, conv, conv.b, dt_bias, A_log, D, norm, o}``), whose
  convolution window and recurrent state live in the request's state slot;
* ``attention``: a `PagedAttention` with grouped-query heads, a weighted RMS norm of every query and key head in
  front of the rotation (``l<i>.mix.{q,k}.norm``), half-split rotary pairs on the first ``rot.dims`` elements, values
  rotated by their own position and outputs turned back, soft-capped scores and a sliding window
  (``l<i>.mix.{q,k,v,o}``);
* ``dense``: the gated feed-forward ``down(silu(gate x) * up x)`` (``l<i>.mlp.{gate,up,down}``);
* ``moe``: `RoutedExperts` with sigmoid scores on the experts' inputs (``l<i>.mlp.router``, ``l<i>.mlp.e<k>.*``) and
  an optional shared expert (``l<i>.mlp.shared.*``).

``final.norm`` (grouped like the others), ``head``, and a soft cap on the logits.
"""

from __future__ import annotations

from slipstream_b200.config.fokedra_config import RotaryConfig
from slipstream_b200.config.sarudra_config import SarudraConfig
from slipstream_b200.parts import (BranchNormBlock, GroupRMSNorm, LMHead, NoPositionEncoding, PagedAttention,
                                   RotaryEncoding, RoutedExperts, StateSpaceMixer, SwiGLUFeedForward, TokenEmbedding)

from .decoder import DecoderLM


def _rotary(rot: RotaryConfig | None, head_dim: int, made: dict):
    """One encoding object per distinct rotation (layers that rotate alike share the table)."""
    key = (rot, head_dim)
    if key not in made:
        made[key] = NoPositionEncoding() if rot is None else RotaryEncoding(head_dim, rot.base, rot.dims, exact_table=True)
    return made[key]


def _gated_unit(prefix: str, width: int, ff: int) -> SwiGLUFeedForward:
    return SwiGLUFeedForward(prefix, width, ff, bias=False,
                             names={role: f"{prefix}.{role}" for role in ("gate", "up", "down")})


def build_sarudra(config: SarudraConfig) -> DecoderLM:
    c = config
    blocks, rotaries = [], {}

    def norm(name: str) -> GroupRMSNorm:
        return GroupRMSNorm(name, c.hidden_size, c.norm_eps, c.norm_groups, tensor=name)

    for i, layer in enumerate(c.layers):
        p, m = f"l{i}", layer.mixer
        if layer.type == "attention":
            mixer = PagedAttention(
                f"{p}.mix", c.hidden_size, m.heads, m.kv_heads, m.dim, _rotary(m.rot, m.dim, rotaries), qkv_bias=False,
                out_bias=False, window=m.window, scale=m.scale, value_dim=m.vdim, qk_norm_eps=c.norm_eps,
                rotate_values=m.rot is not None, softcap=m.softcap,
                names={**{role: f"{p}.mix.{role}" for role in "qkvo"}, "q_norm": f"{p}.mix.q.norm",
                       "k_norm": f"{p}.mix.k.norm"})
        else:
            mixer = StateSpaceMixer(
                f"{p}.mix", c.hidden_size, m.heads, m.vdim, m.state, m.groups, m.conv, m.norm_groups, c.norm_eps,
                names={"in": f"{p}.mix.in", "conv": f"{p}.mix.conv", "conv_bias": f"{p}.mix.conv.b",
                       "dt_bias": f"{p}.mix.dt_bias", "a_log": f"{p}.mix.A_log", "d": f"{p}.mix.D",
                       "norm": f"{p}.mix.norm", "out": f"{p}.mix.o"})
        ffn = None
        if layer.mlp is not None and layer.mlp.kind == "dense":
            ffn = _gated_unit(f"{p}.mlp", c.hidden_size, layer.mlp.ff)
        elif layer.mlp is not None:
            shared = _gated_unit(f"{p}.mlp.shared", c.hidden_size, layer.mlp.shared_ff) if layer.mlp.shared_ff else None
            ffn = RoutedExperts(f"{p}.mlp", c.hidden_size, layer.mlp.ff, layer.mlp.experts, layer.mlp.top, shared=shared,
                                renormalize=False, weight_on_input=True, router_tensor=f"{p}.mlp.router",
                                expert_names=f"{p}.mlp.e{{e}}.{{role}}")
        blocks.append(BranchNormBlock(mixer, ffn, norm(f"{p}.norm1"), norm(f"{p}.norm2") if ffn is not None else None))
    return DecoderLM(
        c,
        TokenEmbedding("embed", c.vocab_size, c.hidden_size, scale=c.embedding_scale, tensor="embed"),
        blocks,
        norm("final.norm"),
        LMHead("head", c.vocab_size, c.hidden_size, tied_to=None, tensor="head", softcap=c.logit_softcap))
