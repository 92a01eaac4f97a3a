"""Building blocks of hybrid decoders: a short causal convolution with a carried tail, linear recurrences
with an fp32 state (constant decay per head, or the selective state-space form), the gated norms that follow
them, and causal softmax attention whose key and value sizes may differ.

Every block reads the step's ``Context`` (which tokens belong to which sequence, their cache slots and
state slots) and runs on the kernels of ``csrc/seq_ops.cu`` / ``csrc/seq_mixers.cu``. Per-sequence state is
NOT owned by the blocks: a block declares what it needs per sequence (``state_shapes``), the runner
allocates one row per state slot and binds it, and the scheduler's block manager hands slots to sequences.
A span that starts at position 0 ignores what its slot held, so slots need no clearing when reused.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..utils.context import get_context

F32 = torch.float32


def small_param(*shape, fill: float = 0.0) -> nn.Parameter:
    """fp32 whatever the model dtype: norm weights, taps, decays and biases enter fp32 arithmetic."""
    return nn.Parameter(torch.full(shape, fill, dtype=F32))


def _spans_and_slots(module_state):
    ctx = get_context()
    spans = ops.StepSpans.of(ctx)
    bound = module_state is not None and module_state.numel() > 0 and ctx.state_slots is not None
    return ctx, spans, bound


class ShortConv(nn.Module):
    """y_t = act(b + sum_j w[:, j] * u_(t - taps + 1 + j)) per channel; ``conv_state`` keeps each sequence's
    last taps - 1 inputs. Channels may be the concatenation of several projections (``segments``), each loaded
    from its own checkpoint tensor."""

    def __init__(self, segments, taps: int, bias: bool = False, act: str | None = None):
        super().__init__()
        self.segments = list(segments)
        self.channels, self.taps, self.act = sum(self.segments), int(taps), act
        self.weight = small_param(self.channels, self.taps)
        self.weight.weight_loader = self._load_segment
        if bias:
            self.bias = small_param(self.channels)
            self.bias.weight_loader = self._load_segment
        else:
            self.register_parameter("bias", None)
        self.conv_state = None

    def _load_segment(self, param, loaded, shard_id: int = 0):
        start = sum(self.segments[:shard_id])
        param.data.narrow(0, start, loaded.shape[0]).copy_(loaded)

    def state_shapes(self):
        return {"conv_state": ((self.taps - 1, self.channels), None)} if self.taps > 1 else {}

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ctx, spans, bound = _spans_and_slots(self.conv_state)
        return ops.causal_conv(x, self.weight, self.bias, spans, self.conv_state if bound else None,
                               ctx.state_slots if bound else None, self.act)


class LinearRecurrence(nn.Module):
    """o_t = S_t^T q_t with S_t = a_t S_(t-1) + k_t (b_t v_t)^T per head, S fp32 [kdim, vdim] in ``state``.
    ``decay`` (a list, one constant per head) selects the constant-decay form; otherwise the selective form
    with learned ``dt_bias``, ``A_log`` and ``D`` (a_t = exp(-exp(A_log) softplus(dt_t + dt_bias)))."""

    def __init__(self, num_heads: int, groups: int, kdim: int, vdim: int, decay=None, act_silu: bool = False):
        super().__init__()
        self.num_heads, self.groups, self.kdim, self.vdim = num_heads, groups, kdim, vdim
        self.act_silu = act_silu
        if decay is not None:
            self.register_buffer("decay", torch.tensor([float(d) for d in decay], dtype=F32), persistent=False)
            assert self.decay.numel() == num_heads, "one decay per head"
        else:
            self.decay = None
            self.dt_bias, self.A_log, self.D = small_param(num_heads), small_param(num_heads), small_param(num_heads)
        self.state = None

    def state_shapes(self):
        return {"state": ((self.num_heads, self.kdim, self.vdim), F32)}

    def forward(self, q, k, v, dt=None) -> torch.Tensor:
        ctx, spans, bound = _spans_and_slots(self.state)
        kw = dict(decay=self.decay, act_silu=self.act_silu) if self.decay is not None else dict(
            dt=dt, dt_bias=self.dt_bias, a_log=self.A_log, d_skip=self.D)
        return ops.linear_recurrence(q, k, v, spans, self.num_heads, self.groups, self.kdim, self.vdim,
                                     self.state if bound else None, ctx.state_slots if bound else None, **kw)


class GatedNorm(nn.Module):
    """RMS norm over ``groups`` equal parts of the row times a plain weight, and a gate act(g): the gate is
    applied before the norm (``gate_first``) or after it. ``norm=False``: the gate alone."""

    def __init__(self, size: int, eps: float, groups: int = 1, gate_first: bool = False, gate_act: str = "sigmoid",
                 norm: bool = True):
        super().__init__()
        self.eps, self.groups, self.gate_first, self.gate_act = eps, groups, gate_first, gate_act
        if norm:
            self.weight = small_param(size, fill=1.0)
        else:
            self.register_parameter("weight", None)

    def forward(self, y: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
        return ops.gated_norm(y, gate, self.weight, self.eps, self.groups, self.gate_first, self.gate_act)


class VarSizeAttention(nn.Module):
    """Causal softmax attention with ``dim``-wide queries/keys and ``vdim``-wide values over paged caches
    ``k_cache`` [nb, bs, G*dim] / ``v_cache`` [nb, bs, G*vdim] (bound by the runner; K/V rows are written by the
    caller's fused epilogue). 16-bit models with dim == vdim in {64, 128} run on the tcgen05 prefill kernel and
    the paged decode kernel of the dense decoders; everything else (other sizes, fp32) on the generic kernel."""

    def __init__(self, num_heads: int, num_kv_heads: int, dim: int, vdim: int, scale: float):
        super().__init__()
        self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.scale = num_heads, num_kv_heads, dim, vdim, scale
        self.k_cache = torch.tensor([])
        self.v_cache = torch.tensor([])
        self.layer_id = -1
        self.force_generic = False

    def cache_rows(self) -> tuple[int, int]:
        return self.num_kv_heads * self.dim, self.num_kv_heads * self.vdim

    def _fast(self, q) -> bool:
        rep, G = self.num_heads // self.num_kv_heads, self.num_kv_heads
        return (not self.force_generic and q.dtype in (torch.bfloat16, torch.float16) and self.dim == self.vdim
                and self.dim in (64, 128) and rep <= 8 and (G in (1, 2, 4) or G % 8 == 0))

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """q [T, H, dim]; k [T, G, dim], v [T, G, vdim]: this step's rows (used when no cache is bound)."""
        ctx = get_context()
        paged = self.k_cache.numel() > 0 and ctx.block_tables is not None
        if self._fast(q) and (paged or ctx.is_prefill):
            if not ctx.is_prefill:
                return ops.paged_decode_attn(q, self.k_cache, self.v_cache, ctx.block_tables, ctx.context_lens,
                                             self.scale, self.num_kv_heads, num_ctas=ctx.decode_attn_ctas)
            if paged and ctx.block_size % 16 == 0:
                return ops.prefill_varlen_attn(q, self.k_cache, self.v_cache, ctx.cu_seqlens_q, ctx.cu_seqlens_k,
                                               ctx.max_seqlen_q, ctx.max_seqlen_k, self.scale, self.num_kv_heads,
                                               block_tables=ctx.block_tables)
            if not paged:
                return ops.prefill_varlen_attn(q, k, v, ctx.cu_seqlens_q, ctx.cu_seqlens_k, ctx.max_seqlen_q,
                                               ctx.max_seqlen_k, self.scale, self.num_kv_heads)
        spans = ops.StepSpans.of(ctx)
        if paged:
            return ops.attn_generic(q, self.k_cache, self.v_cache, spans, self.scale, self.num_kv_heads, self.vdim,
                                    block_tables=ctx.block_tables)
        return ops.attn_generic(q, k, v, spans, self.scale, self.num_kv_heads, self.vdim)
