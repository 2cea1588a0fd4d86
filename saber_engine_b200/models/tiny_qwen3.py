"""Tiny Qwen3-style decoder on the CPU (fp32): the plumbing configuration.  Two layers, hidden 256,
4 query / 2 KV heads of 64, RoPE theta 1e6, RMSNorm eps 1e-6, SwiGLU 768, vocab 1024, tied
embeddings, random-init N(0, 0.02) from a seed.  It runs through the REAL scheduler, allocators and
paged KV cache (page 16) with a CPU executor; `forward_full` is the cache-free oracle.

The reference has no whole-model CPU forward (its CPU code is the expert-chain twin, the sampler,
draft verification and pack tools), so this oracle is a plain restatement of the architecture and
is also the timed CPU baseline of that configuration.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as Fn

from ..sched.executor import SeqOut, SeqRun
from .config import TinyQwen3Config


class TinyQwen3:
    def __init__(self, cfg: Optional[TinyQwen3Config] = None, seed: int = 0, n_blocks: int = 512):
        self.cfg = cfg or TinyQwen3Config()
        c = self.cfg
        g = torch.Generator().manual_seed(seed)
        r = lambda *s: torch.randn(*s, generator=g) * 0.02          # noqa: E731
        self.embed = r(c.vocab, c.hidden)
        self.layers = []
        for _ in range(c.n_layers):
            self.layers.append(dict(
                in_norm=torch.ones(c.hidden), post_norm=torch.ones(c.hidden),
                wq=r(c.n_q_heads * c.head_dim, c.hidden), wk=r(c.n_kv_heads * c.head_dim, c.hidden),
                wv=r(c.n_kv_heads * c.head_dim, c.hidden), wo=r(c.hidden, c.n_q_heads * c.head_dim),
                q_norm=torch.ones(c.head_dim), k_norm=torch.ones(c.head_dim),
                gate=r(c.ffn_inter, c.hidden), up=r(c.ffn_inter, c.hidden), down=r(c.hidden, c.ffn_inter)))
        self.final_norm = torch.ones(c.hidden)
        self.n_blocks = n_blocks
        # paged KV: [layer][block][kv head][2][page][head_dim]
        self.kv = torch.zeros(c.n_layers, n_blocks, c.n_kv_heads, 2, c.page_tokens, c.head_dim)

    # ---- pieces
    def _norm(self, x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.cfg.eps) * w

    def _rope(self, x, pos):
        """x [T, heads, D], pos [T]; rotate-half over the full head."""
        D = x.shape[-1]
        inv = self.cfg.rope_theta ** (-torch.arange(0, D, 2, dtype=torch.float32) / D)
        ang = pos.float()[:, None] * inv[None, :]
        cs, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        a, b = x[..., : D // 2], x[..., D // 2:]
        return torch.cat([a * cs - b * sn, b * cs + a * sn], -1)

    def _attend(self, q, k, v, q_pos):
        """q [T, nq, D]; k, v [S, nkv, D]; causal by absolute position (keys are positions 0..S-1)."""
        c = self.cfg
        g = c.n_q_heads // c.n_kv_heads
        kk, vv = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
        s = torch.einsum("thd,shd->hts", q, kk) / math.sqrt(c.head_dim)
        mask = torch.arange(k.shape[0])[None, :] <= q_pos[:, None]
        s = s.masked_fill(~mask[None], float("-inf"))
        return torch.einsum("hts,shd->thd", torch.softmax(s, -1), vv)

    def _layer(self, h, lw, pos, kv_fn):
        c = self.cfg
        T = h.shape[0]
        x = self._norm(h, lw["in_norm"])
        q = (x @ lw["wq"].t()).reshape(T, c.n_q_heads, c.head_dim)
        k = (x @ lw["wk"].t()).reshape(T, c.n_kv_heads, c.head_dim)
        v = (x @ lw["wv"].t()).reshape(T, c.n_kv_heads, c.head_dim)
        q = self._rope(self._norm(q, lw["q_norm"]), pos)
        k = self._rope(self._norm(k, lw["k_norm"]), pos)
        k_all, v_all = kv_fn(k, v)
        a = self._attend(q, k_all, v_all, pos).reshape(T, -1)
        h = h + a @ lw["wo"].t()
        x = self._norm(h, lw["post_norm"])
        return h + (Fn.silu(x @ lw["gate"].t()) * (x @ lw["up"].t())) @ lw["down"].t()

    # ---- cache-free oracle
    @torch.no_grad()
    def forward_full(self, ids: list) -> torch.Tensor:
        pos = torch.arange(len(ids))
        h = self.embed[torch.tensor(ids)]
        for lw in self.layers:
            h = self._layer(h, lw, pos, lambda k, v: (k, v))
        return self._norm(h, self.final_norm) @ self.embed.t()

    @torch.no_grad()
    def greedy_reference(self, prompt: list, n: int) -> list:
        ids, out = list(prompt), []
        for _ in range(n):
            t = int(self.forward_full(ids)[-1].argmax())
            out.append(t)
            ids.append(t)
        return out

    # ---- paged step
    @torch.no_grad()
    def forward_paged(self, tokens: list, pos0: int, blocks: list) -> torch.Tensor:
        """Rows [pos0, pos0 + T) of one sequence through the paged cache; returns logits [T, vocab]."""
        c = self.cfg
        T = len(tokens)
        pos = torch.arange(pos0, pos0 + T)
        blk = torch.tensor(blocks)
        page = c.page_tokens
        h = self.embed[torch.tensor(tokens)]
        for li, lw in enumerate(self.layers):
            def kv_fn(k, v, li=li):
                b, o = blk[pos // page], pos % page
                self.kv[li, b, :, 0, o] = k
                self.kv[li, b, :, 1, o] = v
                S = pos0 + T
                nb = (S + page - 1) // page
                pages = self.kv[li, blk[:nb]]                     # [nb, nkv, 2, page, D]
                k_all = pages[:, :, 0].permute(0, 2, 1, 3).reshape(nb * page, c.n_kv_heads, c.head_dim)[:S]
                v_all = pages[:, :, 1].permute(0, 2, 1, 3).reshape(nb * page, c.n_kv_heads, c.head_dim)[:S]
                return k_all, v_all
            h = self._layer(h, lw, pos, kv_fn)
        return self._norm(h, self.final_norm) @ self.embed.t()


class TinyExecutor:
    """StepExecutor over TinyQwen3. No drafter: verify width 1 (plus an optional prompt-lookup
    drafter supplied by the caller through `draft_fn`)."""

    def __init__(self, model: Optional[TinyQwen3] = None, max_seqs: int = 8, draft_fn=None, widths=(1,)):
        self.model = model or TinyQwen3()
        c = self.model.cfg
        self.max_seqs, self.page_tokens, self.vocab = max_seqs, c.page_tokens, c.vocab
        self.n_kv_blocks = self.model.n_blocks
        self.decode_batches = tuple(range(1, max_seqs + 1))
        self.decode_widths = tuple(widths)
        self.prefill_rungs = (64, 256, 1024)
        self.draft_fn = draft_fn
        self.history = {}          # slot -> committed token ids (for the lookup drafter)

    def reset_slot(self, slot: int) -> None:
        self.history[slot] = []

    def _drafts(self, slot: int, k: int) -> list:
        return self.draft_fn(self.history[slot], k) if self.draft_fn and k > 0 else []

    def prefill(self, runs: list) -> list:
        outs = []
        for r in runs:
            logits = self.model.forward_paged(r.tokens, r.pos0, r.blocks)
            self.history[r.slot] = self.history.get(r.slot, [])[: r.pos0] + list(r.tokens)
            if r.last_chunk:
                tok = int(logits[-1].argmax())
                self.history[r.slot].append(tok)
                outs.append(SeqOut([tok], self._drafts(r.slot, max(self.decode_widths) - 1), logits_rows=logits[-1:]))
                self.history[r.slot].pop()
            else:
                outs.append(SeqOut([]))
        return outs

    def decode(self, runs: list, width: int) -> list:
        outs = []
        for r in runs:
            logits = self.model.forward_paged(r.tokens, r.pos0, r.blocks)
            picks = logits.argmax(-1).tolist()
            a = 0
            while a < width - 1 and r.tokens[a + 1] == picks[a]:
                a += 1
            toks = picks[: a + 1]
            hist = self.history.get(r.slot, [])[: r.pos0] + list(r.tokens[: a + 1])
            self.history[r.slot] = hist + [toks[-1]]
            drafts = self._drafts(r.slot, width - 1)
            self.history[r.slot] = hist
            outs.append(SeqOut(toks, drafts, logits_rows=logits[: a + 1]))
        return outs

    def snapshot_state(self, slot: int):
        return list(self.history.get(slot, []))

    def restore_state(self, slot: int, snap) -> None:
        self.history[slot] = list(snap)

    def snapshot_bytes(self) -> int:
        return 4096

    def free_snapshot(self, snap) -> None:
        pass
