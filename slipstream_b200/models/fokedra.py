"""Builder of the Fokedra decoder from ``FokedraConfig``: which parts stand in which layer, with which constants
and tensor names.

Per layer ``l<i>``: a `PagedAttention` mixer (grouped-query heads, neighbouring-pair rotary positions on the
first ``rot.dims`` elements with YaRN-stretched frequencies, a weightless RMS norm of every query and key head
after the rotation, a score scale from the configuration, a chunked causal mask, a sigmoid gate on the
concatenated heads; tensors ``l<i>.mix.{q,k,v,g,o}``) and, unless ``mlp`` is null, a gated feed-forward
``g sigmoid(1.702 g) (u + 1)`` with clamped inputs (``l<i>.mlp.{gate,up,down}``), each behind an RMS norm
(``l<i>.norm1``, ``l<i>.norm2``) and joined to the residual streams by hyper-connections (``l<i>.hc1.*``,
``l<i>.hc2.*``).  A layer whose mixer names ``kv_from`` has no key/value projections: its entry in the model's
order reads the pages of the named layer.  ``final.norm`` over the sum of the streams, then ``head``.
"""

from __future__ import annotations

from slipstream_b200.config.fokedra_config import FokedraConfig, RotaryConfig
from slipstream_b200.parts import (ConnectedNorm, HyperConnectionBlock, LMHead, NoPositionEncoding, PagedAttention,
                                   RotaryEncoding, GatedFeedForward, TokenEmbedding, YarnRotaryEncoding)

from .decoder import DecoderLM, ExecEntry

GATE_STEEPNESS = 1.702  # the feed-forward's gate is g * sigmoid(1.702 g) ...
UP_SHIFT = 1.0          # ... times (u + 1)


def _rotary(rot: RotaryConfig | None, head_dim: int, made: dict):
    """One encoding object per distinct rotation (layers that rotate alike share the table)."""
    if rot not in made:
        if rot is None:
            made[rot] = NoPositionEncoding()
        elif rot.scaling is None:
            made[rot] = RotaryEncoding(head_dim, rot.base, rot.dims, interleaved=True, exact_table=True)
        else:
            factor, original, fast, slow = rot.scaling
            made[rot] = YarnRotaryEncoding(head_dim, rot.base, rot.dims, interleaved=True, factor=factor,
                                           original=original, fast=fast, slow=slow)
    return made[rot]


def build_fokedra(config: FokedraConfig) -> DecoderLM:
    c = config
    streams = c.streams or 1
    connected = c.streams is not None  # without the key there are no connection tensors: the plain residual sum
    blocks, order, rotaries = [], [], {}
    for i, layer in enumerate(c.layers):
        p, m = f"l{i}", layer.mixer
        attention = PagedAttention(
            f"{p}.mix", c.hidden_size, m.heads, m.kv_heads, m.dim, _rotary(m.rot, m.dim, rotaries), qkv_bias=False,
            out_bias=False, scale=m.scale, chunk=m.chunk, value_dim=m.vdim, unit_norm_eps=c.norm_eps, gate=True,
            has_kv=m.kv_from is None, names={role: f"{p}.mix.{role}" for role in "qkvgo"})
        ffn = ffn_norm = None
        if layer.mlp is not None:
            ffn = GatedFeedForward(f"{p}.mlp", c.hidden_size, layer.mlp.ff, bias=False, alpha=GATE_STEEPNESS,
                                   limit=layer.mlp.limit, up_shift=UP_SHIFT,
                                   names={role: f"{p}.mlp.{role}" for role in ("gate", "up", "down")})
            ffn_norm = ConnectedNorm(f"{p}.norm2", c.hidden_size, c.norm_eps, streams, f"{p}.hc2" if connected else None)
        blocks.append(HyperConnectionBlock(
            attention, ffn, ConnectedNorm(f"{p}.norm1", c.hidden_size, c.norm_eps, streams, f"{p}.hc1" if connected else None),
            ffn_norm))
        order.append(ExecEntry(i, cache_of=m.kv_from))  # layer j is entry j of the order
    return DecoderLM(
        c,
        TokenEmbedding("embed", c.vocab_size, c.hidden_size, scale=c.embedding_scale, copies=streams, tensor="embed"),
        blocks,
        ConnectedNorm("final.norm", c.hidden_size, c.norm_eps, streams, None),
        LMHead("head", c.vocab_size, c.hidden_size, tied_to=None, tensor="head"),
        order=order)
