"""Zegopel: a decoder whose layers are listed one by one in its configuration, each with one of three
sequence mixers and an optional gated feed-forward, on an fp32 residual stream with a norm before AND after
every sublayer.

    r <- r + N_post(mixer(N_pre(r)));   r <- r + N_post'(ff(N_pre'(r)))      N(x) = x / rms(x) * (1 + w)

  attention   q, k, v projections with bias -> short causal convolution over time on every channel -> q and k
              divided by their per-head root mean square -> q times 1 + c ln(floor((p + 1) / m) + 1) at position
              p -> causal softmax(scale q.k) over the paged cache (no rotation) -> times sigmoid(W_g h) -> W_o
  lightning   q, k, v = silu(projections); per head S <- decay S + k v^T, o = S^T q; RMS norm over all heads,
              times sigmoid(W_g h) -> W_o
  mamba2      one projection into [z | x | B | C | dt]; causal convolution + silu on x, B, C; selective
              state-space recurrence per head with step softplus(dt + bias); times silu(z); grouped RMS norm -> W_o

Launches per sublayer: one GEMM in (all projections of the mixer fused), the convolution, one fused epilogue
(unit norms + temperature + K/V scatter), the mixer kernel, the gate/norm kernel, one GEMM out, and ONE kernel
for "post-norm, residual add, next pre-norm" -- the counterpart of the dense decoders' fused add+RMSNorm.
What the design fixes is a constant here; every size and every constant that may differ between models comes from the config.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

from .. import ops
from ..layers.embed_head import ParallelLMHead, VocabParallelEmbedding
from ..layers.linear import MergedColumnParallelLinear, ReplicatedLinear, RowParallelLinear, tp_rank_size
from ..layers.seq_mixers import (GatedNorm, LinearRecurrence, ShortConv, VarSizeAttention, small_param)
from ..utils.context import get_context

NORM_OFFSET = 1.0          # norm weights of the residual path are stored as deviations from one
FF_ACT = "relu"


@dataclass
class ZegopelSpec:
    """What the runner asks of a model's spec."""
    vocab_size: int
    hidden_size: int
    num_layers: int
    rms_eps: float
    num_experts: int = 0
    tie_embeddings: bool = False


class OffsetNorm(nn.Module):
    """Weight of one norm of the residual path; the arithmetic runs in the fused residual kernels."""

    def __init__(self, size: int):
        super().__init__()
        self.weight = small_param(size)


class AttentionMixer(nn.Module):

    def __init__(self, width: int, m: dict, eps: float):
        super().__init__()
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        self.H, self.G, self.d, self.dv, self.eps = H, G, d, dv, eps
        self.temp_coef, self.temp_every = float(m["q_temp"]["coef"]), int(m["q_temp"]["every"])
        self.sizes = [H * d, G * d, G * dv, H * dv]                     # q | k | v | gate
        self.proj = MergedColumnParallelLinear(width, self.sizes, bias=True)
        self.conv = ShortConv(self.sizes[:3], m["conv"])
        self.attn = VarSizeAttention(H, G, d, dv, float(m["scale"]))
        self.gate = GatedNorm(H * dv, eps, norm=False)
        self.o_proj = RowParallelLinear(H * dv, width)

    def forward(self, positions, h):
        qkvg = self.proj(h)
        nq, nk, nv = self.sizes[:3]
        qkv = self.conv(qkvg[:, :nq + nk + nv])
        attn = self.attn
        ctx = get_context()
        have_cache = attn.k_cache.numel() > 0 and ctx.slot_mapping is not None
        ops.unitnorm_temp_cache(qkv, positions, self.eps, self.temp_coef, self.temp_every, self.H, self.G, self.d,
                                self.dv, attn.k_cache if have_cache else None, attn.v_cache if have_cache else None,
                                ctx.slot_mapping if have_cache else None)
        q = qkv[:, :nq].unflatten(1, (self.H, self.d))
        k = qkv[:, nq:nq + nk].unflatten(1, (self.G, self.d))
        v = qkv[:, nq + nk:].unflatten(1, (self.G, self.dv))
        o = attn(q, k, v)
        return self.o_proj(self.gate(o, qkvg[:, nq + nk + nv:]))


class LightningMixer(nn.Module):

    def __init__(self, width: int, m: dict, eps: float):
        super().__init__()
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        self.sizes = [H * d, H * d, H * dv, H * dv]                     # q | k | v | gate
        self.proj = MergedColumnParallelLinear(width, self.sizes)
        self.rec = LinearRecurrence(H, H, d, dv, decay=m["decay"], act_silu=True)
        self.norm = GatedNorm(H * dv, eps, gate_first=False, gate_act="sigmoid")
        self.o_proj = RowParallelLinear(H * dv, width)

    def forward(self, positions, h):
        p = self.proj(h)
        nq, nk, nv, _ = self.sizes
        o = self.rec(p[:, :nq], p[:, nq:nq + nk], p[:, nq + nk:nq + nk + nv])
        return self.o_proj(self.norm(o, p[:, nq + nk + nv:]))


class Mamba2Mixer(nn.Module):

    def __init__(self, width: int, m: dict, eps: float):
        super().__init__()
        H, dv, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
        self.inner, self.bc = H * dv, G * N
        self.in_proj = ReplicatedLinear(width, 2 * self.inner + 2 * self.bc + H)      # z | x | B | C | dt
        self.conv = ShortConv([self.inner + 2 * self.bc], m["conv"], bias=True, act="silu")
        self.rec = LinearRecurrence(H, G, N, dv)
        self.norm = GatedNorm(self.inner, eps, groups=m["norm_groups"], gate_first=True, gate_act="silu")
        self.o_proj = RowParallelLinear(self.inner, width)

    def forward(self, positions, h):
        p = self.in_proj(h)
        inner, bc = self.inner, self.bc
        xbc = self.conv(p[:, inner:2 * inner + 2 * bc])
        y = self.rec(xbc[:, inner + bc:], xbc[:, inner:inner + bc], xbc[:, :inner], dt=p[:, 2 * inner + 2 * bc:])
        return self.o_proj(self.norm(y, p[:, :inner]))


class GatedFeedForward(nn.Module):

    def __init__(self, width: int, ff: int, act: str):
        super().__init__()
        self.act = act
        self.gate_up_proj = MergedColumnParallelLinear(width, [ff, ff])
        self.down_proj = RowParallelLinear(ff, width)

    def forward(self, h):
        return self.down_proj(ops.act_and_mul(self.gate_up_proj(h), self.act))


MIXERS = {"attention": AttentionMixer, "lightning": LightningMixer, "mamba2": Mamba2Mixer}


class ZegopelLayer(nn.Module):

    def __init__(self, width: int, entry: dict, eps: float):
        super().__init__()
        if entry["type"] not in MIXERS:
            raise ValueError(f"unknown mixer {entry['type']!r}")
        self.mix = MIXERS[entry["type"]](width, entry["mixer"], eps)
        self.norm1, self.norm1b = OffsetNorm(width), OffsetNorm(width)
        mlp = entry.get("mlp")
        if mlp:
            if mlp.get("kind", "dense") != "dense":
                raise ValueError(f"unknown feed-forward kind {mlp['kind']!r}")
            self.mlp = GatedFeedForward(width, mlp["ff"], mlp.get("act", FF_ACT))
            self.norm2, self.norm2b = OffsetNorm(width), OffsetNorm(width)
        else:
            self.mlp = None


class ZegopelForCausalLM(nn.Module):
    supports_fp32 = True            # every kernel of this stack has a true 32-bit form
    prefix_caching = False          # recurrent state at a prefix's end is not kept, so cached blocks are no use
    split_decode = False

    def __init__(self, config):
        super().__init__()
        if tp_rank_size()[1] != 1:
            raise ValueError("Zegopel runs on one GPU per replica (no tensor-parallel sharding of its mixers)")
        c = config.to_dict() if hasattr(config, "to_dict") else dict(config)
        self.eps = float(c["norm"]["eps"])
        W = c["width"]
        self.spec = ZegopelSpec(c["vocab"], W, len(c["layers"]), self.eps)
        self.embed_tokens = VocabParallelEmbedding(c["vocab"], W)
        self.layers = nn.ModuleList([ZegopelLayer(W, entry, self.eps) for entry in c["layers"]])
        self.norm = OffsetNorm(W)
        self.lm_head = ParallelLMHead(c["vocab"], W)
        for layer in self.layers:                      # the gate rows of a fused projection carry no bias
            if getattr(layer.mix, "proj", None) is not None and layer.mix.proj.bias is not None:
                layer.mix.proj.bias.data.zero_()
        self.trace_layers = None                       # a list: the residual stream after every layer is appended

    # ------------------------------------------------------------------ forward
    def _sublayers(self):
        """(pre-norm, callable, post-norm, closes a layer) in execution order."""
        out = []
        for layer in self.layers:
            out.append((layer.norm1, layer.mix, layer.norm1b, layer.mlp is None))
            if layer.mlp is not None:
                out.append((layer.norm2, lambda pos, h, f=layer.mlp: f(h), layer.norm2b, True))
        return out

    def forward(self, input_ids, positions):
        dtype = self.embed_tokens.weight.dtype
        residual = self.embed_tokens(input_ids).float()
        subs = self._sublayers()
        h = ops.residual_rmsnorm(residual, subs[0][0].weight, self.eps, dtype, NORM_OFFSET)
        for i, (_, fn, post, closes) in enumerate(subs):
            y = fn(positions, h)
            nxt = subs[i + 1][0] if i + 1 < len(subs) else self.norm
            h = ops.residual_add_norms_(y.contiguous(), residual, post.weight, nxt.weight, self.eps, NORM_OFFSET)
            if closes and self.trace_layers is not None:
                self.trace_layers.append(residual.clone())
        return h                                       # already through the final norm

    def compute_logits(self, hidden_states):
        return self.lm_head(hidden_states)

    # ------------------------------------------------------------------ weights
    def route_checkpoint_tensor(self, name: str):
        """Checkpoint tensor name -> (parameter name, shard id or None)."""
        if name == "embed":
            return "embed_tokens.weight", None
        if name == "head":
            return "lm_head.weight", None
        if name == "final.norm":
            return "norm.weight", None
        layer, _, rest = name.partition(".")
        i = int(layer[1:])
        base = f"layers.{i}."
        if rest in ("norm1", "norm1b", "norm2", "norm2b"):
            return base + rest + ".weight", None
        if rest.startswith("mlp."):
            key = rest[4:]
            return {"gate": (base + "mlp.gate_up_proj.weight", 0), "up": (base + "mlp.gate_up_proj.weight", 1),
                    "down": (base + "mlp.down_proj.weight", None)}[key]
        key = rest[4:]                                  # after "mix."
        mix = self.layers[i].mix
        if key == "o":
            return base + "mix.o_proj.weight", None
        if isinstance(mix, Mamba2Mixer):
            return {"in": (base + "mix.in_proj.weight", None), "conv": (base + "mix.conv.weight", 0),
                    "conv.b": (base + "mix.conv.bias", 0), "dt_bias": (base + "mix.rec.dt_bias", None),
                    "A_log": (base + "mix.rec.A_log", None), "D": (base + "mix.rec.D", None),
                    "norm": (base + "mix.norm.weight", None)}[key]
        if key == "norm":
            return base + "mix.norm.weight", None
        head, _, tail = key.partition(".")
        shard = "qkvg".index(head)
        if tail == "":
            return base + "mix.proj.weight", shard
        if tail == "b":
            return base + "mix.proj.bias", shard
        if tail == "conv":
            return base + "mix.conv.weight", shard
        raise KeyError(name)

    @torch.no_grad()
    def random_init(self, seed: int = 0, std: float | None = None) -> None:
        """Random weights for synthetic runs: matrices N(0, 1/fan_in), norm deviations and biases small,
        step-size parameters in the range where the recurrences neither vanish nor blow up."""
        g = torch.Generator().manual_seed(seed)
        for name, p in sorted(self.named_parameters()):
            if name.endswith("A_log"):
                v = torch.rand(p.shape, generator=g) * 2 - 2
            elif name.endswith(".D") or name.endswith("mix.norm.weight"):
                v = 1 + 0.1 * torch.randn(p.shape, generator=g)
            elif name.endswith("dt_bias"):
                v = 0.5 * torch.randn(p.shape, generator=g)
            elif name.endswith("conv.weight"):
                v = 0.5 * torch.randn(p.shape, generator=g)
            elif p.dim() == 1:
                v = 0.1 * torch.randn(p.shape, generator=g)
            elif name == "embed_tokens.weight":
                v = torch.randn(p.shape, generator=g)
            else:
                v = torch.randn(p.shape, generator=g) * (std if std is not None else p.shape[1] ** -0.5)
            p.data.copy_(v.to(p.dtype))
        for layer in self.layers:
            if isinstance(layer.mix, AttentionMixer):
                layer.mix.proj.bias.data[sum(layer.mix.sizes[:3]):].zero_()
