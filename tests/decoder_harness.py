"""A small Qwen3-shaped decoder (random weights) whose linear layers run on the tree GEMM, used to check that
greedy decoding is token-identical across tensor-parallel degrees and batch sizes.

Only test infrastructure: it plays the role the vLLM model code plays for the reference's end-to-end check
(simple_inference.py:133-194: same prompts, different (tp, batch) settings, outputs compared).

What is under test is the row-split path: o_proj and down_proj are K-split over `tp` simulated ranks, each
rank's partial comes from `matmul_tp_persistent`, and the partials are combined in the rank-pair tree order
(the arithmetic of the tree all-reduce; its peer-to-peer kernels are checked against the same arithmetic in
tests/test_allreduce_multigpu.py).  The column-split layers (qkv, gate_up, lm_head) use the same GEMM with
the full K, so every output column has the same bits whichever rank computes it.

Everything that is not a GEMM is written so that the kernel shapes a token sees never depend on the batch or
on tp: RMSNorm runs row by row, attention runs per (sequence, head); the remaining ops are elementwise.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from llm_reproducibility_b200.tbik.tree_based_matmul import matmul_tp_persistent


@dataclass
class Config:
    hidden: int = 2048
    q_heads: int = 16
    kv_heads: int = 8
    head_dim: int = 128
    intermediate: int = 4096
    layers: int = 2
    vocab: int = 2048
    rope_theta: float = 1.0e6
    eps: float = 1.0e-6


def qwen3_8b_shape(layers: int = 2, vocab: int = 4096) -> Config:
    """Qwen3-8B's layer shape (hidden 4096, 32 q / 8 kv heads, head_dim 128, intermediate 12288)."""
    return Config(hidden=4096, q_heads=32, kv_heads=8, head_dim=128, intermediate=12288, layers=layers, vocab=vocab)


class Weights:
    def __init__(self, cfg: Config, seed: int = 0, device="cuda"):
        g = torch.Generator(device=device).manual_seed(seed)

        def w(n, k):
            return (torch.randn(n, k, generator=g, device=device) * 0.02).to(torch.bfloat16)

        D, H = cfg.head_dim, cfg.hidden
        self.embed = w(cfg.vocab, H)
        self.lm_head = w(cfg.vocab, H)
        self.final_norm = (1.0 + 0.1 * torch.randn(H, generator=g, device=device)).to(torch.bfloat16)
        self.layers = []
        for _ in range(cfg.layers):
            self.layers.append({
                "ln1": (1.0 + 0.1 * torch.randn(H, generator=g, device=device)).to(torch.bfloat16),
                "ln2": (1.0 + 0.1 * torch.randn(H, generator=g, device=device)).to(torch.bfloat16),
                "wq": w(cfg.q_heads * D, H), "wk": w(cfg.kv_heads * D, H), "wv": w(cfg.kv_heads * D, H),
                "wo": w(H, cfg.q_heads * D),
                "wg": w(cfg.intermediate, H), "wu": w(cfg.intermediate, H),
                "wd": w(H, cfg.intermediate),
            })


def rmsnorm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm, one row per call: the reduction kernel always sees the shape [1, H]."""
    out = torch.empty_like(x)
    wf = weight.float()
    for i in range(x.shape[0]):
        r = x[i:i + 1].float()
        inv = torch.rsqrt(r.pow(2).mean(-1, keepdim=True) + eps)
        out[i:i + 1] = (r * inv * wf).to(x.dtype)
    return out


def rope(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """x: [T, heads, D]; pos: [T].  Elementwise, so invariant."""
    D = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, device=x.device, dtype=torch.float32) / D))
    ang = pos.float()[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x1, x2 = x.float()[..., : D // 2], x.float()[..., D // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


def tree_sum(parts):
    """((0+1)+(2+3))+((4+5)+(6+7)) in the tensors' dtype: the arithmetic of the tree all-reduce."""
    parts = list(parts)
    while len(parts) > 1:
        parts = [parts[i] + parts[i + 1] for i in range(0, len(parts), 2)]
    return parts[0]


def row_parallel(x: torch.Tensor, W: torch.Tensor, tp: int) -> torch.Tensor:
    """x [T, K] @ W[N, K]^T with K split over tp simulated ranks."""
    K = x.shape[1]
    ks = K // tp
    return tree_sum([matmul_tp_persistent(x[:, r * ks:(r + 1) * ks], W[:, r * ks:(r + 1) * ks].t()) for r in range(tp)])


def column_parallel(x: torch.Tensor, W: torch.Tensor, tp: int) -> torch.Tensor:
    """x [T, K] @ W[N, K]^T with N split over tp simulated ranks (results concatenated)."""
    ns = W.shape[0] // tp
    return torch.cat([matmul_tp_persistent(x, W[r * ns:(r + 1) * ns].t()) for r in range(tp)], dim=1)


class Decoder:
    def __init__(self, cfg: Config, weights: Weights, tp: int):
        assert cfg.kv_heads % tp == 0 and cfg.q_heads % tp == 0
        self.cfg, self.w, self.tp = cfg, weights, tp

    def _attention(self, q, k_cache, v_cache, lens_before, new_counts):
        """Per (sequence, head) causal attention over that sequence's cache; shapes depend only on the sequence."""
        cfg = self.cfg
        out = torch.empty_like(q)
        group = cfg.q_heads // cfg.kv_heads
        scale = 1.0 / math.sqrt(cfg.head_dim)
        start = 0
        for b, n_new in enumerate(new_counts):
            total = lens_before[b] + n_new
            for h in range(cfg.q_heads):
                qh = q[start:start + n_new, h].float()                 # [n_new, D]
                kh = k_cache[b][:total, h // group].float()            # [total, D]
                vh = v_cache[b][:total, h // group].float()
                s = (qh @ kh.t()) * scale
                idx = torch.arange(total, device=q.device)[None, :]
                qpos = (lens_before[b] + torch.arange(n_new, device=q.device))[:, None]
                s = s.masked_fill(idx > qpos, float("-inf"))
                out[start:start + n_new, h] = (torch.softmax(s, dim=-1) @ vh).to(q.dtype)
            start += n_new
        return out

    def forward(self, tokens, positions, k_caches, v_caches, lens_before, new_counts):
        """tokens: [T] (all sequences' new tokens, concatenated).  Returns logits of the last new token of each sequence."""
        cfg, tp = self.cfg, self.tp
        D = cfg.head_dim
        x = self.w.embed[tokens]
        for li, L in enumerate(self.w.layers):
            h = rmsnorm_rows(x, L["ln1"], cfg.eps)
            q = column_parallel(h, L["wq"], tp).view(-1, cfg.q_heads, D)
            k = column_parallel(h, L["wk"], tp).view(-1, cfg.kv_heads, D)
            v = column_parallel(h, L["wv"], tp).view(-1, cfg.kv_heads, D)
            q, k = rope(q, positions, cfg.rope_theta), rope(k, positions, cfg.rope_theta)
            start = 0
            for b, n_new in enumerate(new_counts):
                k_caches[li][b][lens_before[b]:lens_before[b] + n_new] = k[start:start + n_new]
                v_caches[li][b][lens_before[b]:lens_before[b] + n_new] = v[start:start + n_new]
                start += n_new
            a = self._attention(q, k_caches[li], v_caches[li], lens_before, new_counts)
            x = x + row_parallel(a.reshape(-1, cfg.q_heads * D), L["wo"], tp)          # o_proj: K split
            h = rmsnorm_rows(x, L["ln2"], cfg.eps)
            act = torch.nn.functional.silu(column_parallel(h, L["wg"], tp).float()) * column_parallel(h, L["wu"], tp).float()
            x = x + row_parallel(act.to(x.dtype), L["wd"], tp)                          # down_proj: K split
        last = torch.cumsum(torch.tensor(new_counts), 0) - 1
        xl = rmsnorm_rows(x[last.to(x.device)], self.w.final_norm, cfg.eps)
        return column_parallel(xl, self.w.lm_head, tp)

    @torch.no_grad()
    def greedy(self, prompts, steps: int, max_len: int = 0):
        """prompts: list of 1-D token tensors.  Returns (generated ids [B, steps], logits of every step [steps, B, V])."""
        cfg = self.cfg
        B = len(prompts)
        max_len = max_len or max(len(p) for p in prompts) + steps
        dev = self.w.embed.device
        kc = [[torch.zeros(max_len, cfg.kv_heads, cfg.head_dim, dtype=torch.bfloat16, device=dev) for _ in range(B)]
              for _ in range(cfg.layers)]
        vc = [[torch.zeros_like(kc[0][0]) for _ in range(B)] for _ in range(cfg.layers)]
        lens = [0] * B
        tokens = torch.cat(prompts).to(dev)
        pos = torch.cat([torch.arange(len(p)) for p in prompts]).to(dev)
        counts = [len(p) for p in prompts]
        out_ids, out_logits = [], []
        for _ in range(steps):
            logits = self.forward(tokens, pos, kc, vc, lens, counts)
            lens = [a + b for a, b in zip(lens, counts)]
            nxt = logits.float().argmax(-1)
            out_ids.append(nxt)
            out_logits.append(logits)
            tokens, pos, counts = nxt, torch.tensor(lens, device=dev), [1] * B
        return torch.stack(out_ids, 1), torch.stack(out_logits, 0)
