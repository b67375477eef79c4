"""Library baselines written the way a PyTorch user would write them: `torch.nn` modules, bf16 autocast over fp32
parameters, `scaled_dot_product_attention`, `torch.optim` fused optimizers, DistributedDataParallel for several GPUs.
Nothing of this repository's kernels, executors or compiler is on this path; `bench.py --impl torch` times it with the
same synthetic data, the same step contents and the same clock as the framework's own arm.

The Transformer language model mirrors the computation graph the model zoo builds (`transformer_lm`): token embedding,
N post-LayerNorm blocks of (bias-free multi-head self-attention with dropout on the probabilities, residual, LayerNorm,
Linear + ReLU + dropout, Linear + dropout, residual, LayerNorm), a bias-free vocabulary projection and a mean
cross-entropy loss.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
import torch.utils.checkpoint


class Block(nn.Module):
    def __init__(self, d: int, heads: int, ffn: int, p: float, eps: float):
        super().__init__()
        self.h, self.p = heads, p
        self.qkv = nn.Linear(d, 3 * d, bias=False)
        self.proj = nn.Linear(d, d, bias=False)
        self.ln1 = nn.LayerNorm(d, eps=eps)
        self.f1 = nn.Linear(d, ffn)
        self.f2 = nn.Linear(ffn, d)
        self.ln2 = nn.LayerNorm(d, eps=eps)

    def forward(self, x):
        b, s, d = x.shape
        q, k, v = self.qkv(x).view(b, s, 3, self.h, d // self.h).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, dropout_p=self.p if self.training else 0.0)
        x = self.ln1(x + self.proj(a.transpose(1, 2).reshape(b, s, d)))
        f = F.dropout(self.f2(F.dropout(F.relu(self.f1(x)), self.p, self.training)), self.p, self.training)
        return self.ln2(x + f)


class TransformerLM(nn.Module):
    def __init__(self, vocab: int, d: int, heads: int, ffn: int, layers: int, dropout: float, eps: float = 1e-5, init_std: float = 0.02,
                 loss_chunk_rows: int = 8192):
        super().__init__()
        self.emb = nn.Embedding(vocab, d)
        self.blocks = nn.ModuleList(Block(d, heads, ffn, dropout, eps) for _ in range(layers))
        self.head = nn.Linear(d, vocab, bias=False)
        self.loss_chunk_rows = loss_chunk_rows
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, 0.0, init_std)
            if isinstance(m, nn.Linear) and m.bias is not None:
                nn.init.zeros_(m.bias)

    def forward(self, ids, labels):
        """Mean next-token cross entropy.  The vocabulary projection and the loss run over row chunks (each recomputed in
        backward), so the [tokens, vocab] logits never exist as a whole."""
        x = self.emb(ids)
        for blk in self.blocks:
            x = blk(x)
        rows = x.reshape(-1, x.shape[-1])
        tgt = labels.reshape(-1).long()
        total = rows.new_zeros((), dtype=torch.float32)
        for r0 in range(0, rows.shape[0], self.loss_chunk_rows):
            total = total + torch.utils.checkpoint.checkpoint(self._chunk_loss, rows[r0:r0 + self.loss_chunk_rows],
                                                              tgt[r0:r0 + self.loss_chunk_rows], use_reentrant=False)
        return total / rows.shape[0]

    def _chunk_loss(self, rows, tgt):
        return F.cross_entropy(self.head(rows).float(), tgt, reduction="sum")


def build_transformer_lm(cfg: dict) -> TransformerLM:
    return TransformerLM(vocab=cfg["vocab_size"], d=cfg["num_features"], heads=cfg["num_heads"], ffn=cfg["dim_feedforward"],
                         layers=cfg["num_decoder_layers"], dropout=cfg.get("dropout", 0.1), eps=cfg.get("layer_norm_eps", 1e-5),
                         init_std=cfg.get("init_std", 0.02))


def transformer_lm_step_flops(cfg: dict, batch: int) -> float:
    """Multiply-add FLOPs of one training step (forward + backward = 3 x forward GEMM work, attention included)."""
    d, f, s, v, n = cfg["num_features"], cfg["dim_feedforward"], cfg["sequence_length"], cfg["vocab_size"], cfg["num_decoder_layers"]
    tokens = batch * s
    per_layer = 2.0 * tokens * (4 * d * d + 2 * d * f) + 4.0 * tokens * s * d
    return 3.0 * (n * per_layer + 2.0 * tokens * d * v)
