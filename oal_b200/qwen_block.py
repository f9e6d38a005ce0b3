"""Minimal Qwen2.5-0.5B-shaped decoder stack around the operator: the model-level training step.

This is the workload of the reference's experiment reduced to what a step needs
(qwen_lora_experiment/attention/common.py for the layer shell, backbones/spec.py:29-33 for the geometry,
lora.py for rank/alpha on q/k/v/o, kernel_parameters.py for the per-layer group tables and packed
factors): RMSNorm, rotary embedding (theta 1e6), SwiGLU MLP, tied embedding / LM head, frozen random
base weights, trainable LoRA matrices and kernel factors.  Everything except the attention operator is
plain torch (library GEMMs); weights are random and token ids synthetic.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from . import synthetic
from .attention_shell import ModelGeometry, OalAttentionLayer, PreparedCallCache, QWEN_GEOMETRY, rope_tables


class RMSNorm(nn.Module):
    def __init__(self, size: int, eps: float = 1e-6, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(size, dtype=dtype, device=device), requires_grad=False)
        self.eps = eps

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


class SwiGLU(nn.Module):
    def __init__(self, hidden: int, intermediate: int, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.gate = nn.Linear(hidden, intermediate, bias=False, dtype=dtype, device=device)
        self.up = nn.Linear(hidden, intermediate, bias=False, dtype=dtype, device=device)
        self.down = nn.Linear(intermediate, hidden, bias=False, dtype=dtype, device=device)
        for p in self.parameters():
            p.requires_grad_(False)

    def forward(self, x):
        return self.down(F.silu(self.gate(x)) * self.up(x))


class DecoderLayer(nn.Module):
    def __init__(self, layer_id, dim_groups, factor, *, cache, geometry, intermediate, lora_rank, lora_alpha, dtype, device):
        super().__init__()
        self.input_norm = RMSNorm(geometry.hidden_size, dtype=dtype, device=device)
        self.attention = OalAttentionLayer(layer_id, dim_groups, factor, cache=cache, geometry=geometry,
                                           lora_rank=lora_rank, lora_alpha=lora_alpha, dtype=dtype, device=device)
        self.post_norm = RMSNorm(geometry.hidden_size, dtype=dtype, device=device)
        self.mlp = SwiGLU(geometry.hidden_size, intermediate, dtype=dtype, device=device)

    def forward(self, x, position_embeddings):
        x = x + self.attention(self.input_norm(x), position_embeddings)
        return x + self.mlp(self.post_norm(x))


class QwenOalStack(nn.Module):
    """``num_layers`` decoder layers with tied embedding / LM head; forward returns the mean token loss."""

    def __init__(self, *, geometry: ModelGeometry = QWEN_GEOMETRY, num_layers: int | None = None,
                 intermediate: int = 4864, vocab: int = 151936, groups: int = 8, lora_rank: int = 16,
                 lora_alpha: float = 32.0, precision: str = "bf16_tensorcore", seed: int = 0,
                 dtype=torch.bfloat16, device=None):
        super().__init__()
        self.geometry = geometry
        self.cache = PreparedCallCache(precision=precision, output_layout="tokens_first" if precision == "bf16_tensorcore" else "heads_first")
        layers = geometry.num_layers if num_layers is None else num_layers
        gen = torch.Generator().manual_seed(4000 + seed)
        self.embed = nn.Embedding(vocab, geometry.hidden_size, dtype=dtype, device=device)
        self.embed.weight.requires_grad_(False)
        nn.init.normal_(self.embed.weight, std=0.02)
        sizes = synthetic.QWEN_GROUP_SIZES[groups]
        pairs = (groups + 1) * (groups + 2) // 2
        blocks = []
        for layer_id in range(layers):
            # per-head seeded partitions and packed lower-triangular factors with U(0.1, 1) entries
            dim_groups = torch.stack([synthetic.partition_groups(geometry.head_dim, sizes, gen)[0]
                                      for _ in range(geometry.num_query_heads)])
            factor = torch.rand(geometry.num_query_heads, pairs, generator=gen) * 0.9 + 0.1
            blocks.append(DecoderLayer(layer_id, dim_groups.to(device) if device else dim_groups,
                                       factor.to(device) if device else factor, cache=self.cache, geometry=geometry,
                                       intermediate=intermediate, lora_rank=lora_rank, lora_alpha=lora_alpha,
                                       dtype=dtype, device=device))
        self.layers = nn.ModuleList(blocks)
        self.final_norm = RMSNorm(geometry.hidden_size, dtype=dtype, device=device)
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, std=0.02)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)

    def trainable_parameters(self):
        return [p for p in self.parameters() if p.requires_grad]

    def forward(self, token_ids: torch.Tensor, *, loss_chunk: int = 1024):
        b, n = token_ids.shape
        x = self.embed(token_ids)
        position_embeddings = rope_tables(n, self.geometry.head_dim, device=x.device, dtype=x.dtype)
        for layer in self.layers:
            x = layer(x, position_embeddings)
        x = self.final_norm(x)
        # next-token loss through the tied head, in slices of the sequence so that the logits of the whole
        # batch never exist at once
        total = x.new_zeros((), dtype=torch.float32)
        for s in range(0, n - 1, loss_chunk):
            e = min(s + loss_chunk, n - 1)
            logits = x[:, s:e] @ self.embed.weight.t()
            total = total + F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]),
                                            token_ids[:, s + 1:e + 1].reshape(-1), reduction="sum")
        return total / (b * (n - 1))
