"""Model geometry: the dense 27B GDN / gated-attention hybrid, the Flash-Next-style MoE hybrid, the
block drafter and the tiny CPU Qwen3 decoder, plus the per-rank (tensor-parallel) shard shapes.

Parity: dimensions follow the reference's model plane (`crates/saber-model/src/graph.rs:141-160`
ModelConfig::qwen38_27b, `crates/saber-plan/src/model.rs:584-672` per-rank linear shapes,
`crates/saber-model/src/dflash_graph.rs:78-100` drafter, `crates/saber-model/src/qwen4_exp/config.rs:480-518`
Flash-Next).  Unlike the reference, which refuses any TP other than 1 and 2
(`crates/saber-plan/src/model.rs:571-573`), shard rules here cover TP 1/2/4/8: heads divide across
ranks and, where there are fewer KV heads than ranks, each KV head is replicated on tp / n_kv
consecutive ranks.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Optional


@dataclass(frozen=True)
class MoEConfig:
    n_experts: int = 512
    top_k: int = 10
    expert_inter: int = 512
    shared_inter: int = 512
    norm_topk_prob: bool = True
    expert_format: str = "iu8"         # routed experts: "iu8" (int4 x int8 rows) | "mxfp4" (e2m1 / e8m0 per 32, fp8 rows)


@dataclass(frozen=True)
class DrafterConfig:
    """Block drafter: proposes `block` tokens per step from target hidden taps."""
    hidden: int = 5120
    n_layers: int = 5
    inter: int = 4352
    block: int = 8
    n_taps: int = 5            # target layers whose residual stream conditions the drafter
    head_bits: int = 4
    # attention in the first `attn_layers` drafter layers: the block rows attend (causally) over a context-KV
    # store written from the target's last tap row of every context position, and over the block's own rows
    attn_layers: int = 0
    attn_q_heads: int = 4
    attn_kv_heads: int = 1
    attn_window: int = 2048      # sliding window of the drafter's attention (keys a block row sees); 0: the whole context


@dataclass(frozen=True)
class HybridConfig:
    name: str
    n_layers: int
    hidden: int
    n_q_heads: int
    n_kv_heads: int
    head_dim: int
    ffn_inter: int
    vocab: int
    attn_every: int = 4                 # layer i is full attention iff (i + 1) % attn_every == 0
    rot_dim: int = 64
    rope_theta: float = 1e7
    mrope_sections: tuple = (11, 11, 10)
    gdn_k_heads: int = 16
    gdn_v_heads: int = 48
    gdn_head_dim: int = 128
    conv_kernel: int = 4
    eps: float = 1e-6
    norm_offset: float = 1.0            # Gemma-style (1 + w)
    attn_out_gate: bool = True
    tie_embeddings: bool = False
    act_hadamard: bool = False          # rotate activations (sign + 32-point Hadamard) before int8/fp8 quant; weights pre-rotated
    weight_format: str = "iu8"         # 4-bit linears: "iu8" (int4 x int8 acts) | "mxfp4" (e2m1/e8m0 x fp8 acts) | "nvfp4" (native block-scaled FP4 x FP4)
    max_ctx: int = 262144
    page_tokens: int = 16
    moe: Optional[MoEConfig] = None
    drafter: Optional[DrafterConfig] = None
    w8_linears: tuple = ()              # names of the linears kept at int8 (rest int4)
    lm_head_bits: int = 8

    def is_attention_layer(self, i: int) -> bool:
        return self.attn_every > 0 and (i + 1) % self.attn_every == 0

    @property
    def n_attn_layers(self) -> int:
        return sum(self.is_attention_layer(i) for i in range(self.n_layers))

    @property
    def n_gdn_layers(self) -> int:
        return self.n_layers - self.n_attn_layers

    def kv_bytes_per_token(self, tp: int = 1) -> int:
        """fp8 K and V of every attention layer for one token on one rank."""
        sh = shard(self, tp, 0)
        return self.n_attn_layers * sh.n_kv_heads * 2 * self.head_dim

    def gdn_state_bytes_per_seq(self, tp: int = 1, state_bytes: int = 4) -> int:
        sh = shard(self, tp, 0)
        return self.n_gdn_layers * sh.gdn_v_heads * self.gdn_head_dim * self.gdn_head_dim * state_bytes

    def param_count(self) -> int:
        h = self.hidden
        attn = h * (self.n_q_heads * self.head_dim * (2 if self.attn_out_gate else 1)
                    + 2 * self.n_kv_heads * self.head_dim) + self.n_q_heads * self.head_dim * h
        kd, vd = self.gdn_k_heads * self.gdn_head_dim, self.gdn_v_heads * self.gdn_head_dim
        gdn = h * (2 * kd + 2 * vd + 2 * self.gdn_v_heads) + vd * h
        if self.moe:
            mlp = self.moe.n_experts * 3 * h * self.moe.expert_inter + 3 * h * self.moe.shared_inter \
                + h * self.moe.n_experts
        else:
            mlp = 3 * h * self.ffn_inter
        body = self.n_attn_layers * (attn + mlp) + self.n_gdn_layers * (gdn + mlp)
        return body + self.vocab * h * (1 if self.tie_embeddings else 2)


@dataclass(frozen=True)
class ShardShape:
    """Per-rank shapes at a TP degree (N x K of every linear, head counts)."""
    tp: int
    rank: int
    n_q_heads: int
    n_kv_heads: int
    kv_head_first: int        # first global KV head this rank holds
    q_head_first: int
    gdn_k_heads: int
    gdn_v_heads: int
    ffn_inter: int
    vocab: int
    vocab_first: int
    qkv_n: int                # attention merged qkv(+gate) output features
    o_k: int                  # attention o_proj reduction dim
    gdn_in_n: int             # merged q|k|v|z|b|a output features
    gdn_conv_c: int           # conv channels q|k|v
    gdn_out_k: int


def shard(cfg: HybridConfig, tp: int, rank: int) -> ShardShape:
    if tp not in (1, 2, 4, 8):
        raise ValueError(f"tensor-parallel degree {tp} is not supported (1, 2, 4 or 8)")
    if cfg.n_q_heads % tp or cfg.gdn_k_heads % tp or cfg.gdn_v_heads % tp or \
            (cfg.moe is None and cfg.ffn_inter % (tp * 128)) or (cfg.moe is not None and cfg.moe.n_experts % tp):
        raise ValueError(f"{cfg.name}: heads / FFN do not divide by tp={tp}")
    nq = cfg.n_q_heads // tp
    if cfg.n_kv_heads >= tp:
        nkv = cfg.n_kv_heads // tp
        kv_first = rank * nkv
    else:
        nkv = 1
        kv_first = rank * cfg.n_kv_heads // tp    # each KV head lives on tp / n_kv consecutive ranks
    hk, hv = cfg.gdn_k_heads // tp, cfg.gdn_v_heads // tp
    d = cfg.gdn_head_dim
    vocab = (cfg.vocab + tp - 1) // tp
    gate = 2 if cfg.attn_out_gate else 1
    return ShardShape(
        tp=tp, rank=rank, n_q_heads=nq, n_kv_heads=nkv, kv_head_first=kv_first, q_head_first=rank * nq,
        gdn_k_heads=hk, gdn_v_heads=hv, ffn_inter=cfg.ffn_inter // tp,
        vocab=min(vocab, cfg.vocab - rank * vocab), vocab_first=rank * vocab,
        qkv_n=nq * cfg.head_dim * gate + 2 * nkv * cfg.head_dim, o_k=nq * cfg.head_dim,
        gdn_in_n=2 * hk * d + 2 * hv * d + 2 * hv, gdn_conv_c=2 * hk * d + hv * d, gdn_out_k=hv * d)


# The 19 row-parallel linears the W4A8-iu8 pack keeps at int8 ("which ones is pack data"); the
# synthetic pack promotes the first and last layers' reduction-side linears and every eighth down_proj.
def default_w8_set(n_layers: int) -> tuple:
    names = []
    for i in (0, 1, n_layers - 2, n_layers - 1):
        names += [f"layers.{i}.mixer.out", f"layers.{i}.mlp.down"]
    for i in range(4, n_layers - 2, 6):
        names.append(f"layers.{i}.mlp.down")
    names = list(dict.fromkeys(names))
    i = 2
    while len(names) < 19 and i < n_layers:
        n = f"layers.{i}.mixer.out"
        if n not in names:
            names.append(n)
        i += 3
    return tuple(names[:19])


def qwen38_27b() -> HybridConfig:
    return HybridConfig(
        name="qwen38-27b", n_layers=64, hidden=5120, n_q_heads=24, n_kv_heads=4, head_dim=256,
        ffn_inter=17408, vocab=248320, rope_theta=1e7, drafter=DrafterConfig(),
        w8_linears=default_w8_set(64))


def flashnext_moe(reference_geometry: bool = False) -> HybridConfig:
    """Flash-Next-style MoE hybrid. Default = the benchmark geometry; reference_geometry=True gives
    the reference's 2560 / 640 / 248,320 dimensions (without hyper-connections, PLE, QSA, MTP)."""
    if reference_geometry:
        return HybridConfig(
            name="flashnext-ref", n_layers=48, hidden=2560, n_q_heads=24, n_kv_heads=2, head_dim=256,
            ffn_inter=640, vocab=248320,
            moe=MoEConfig(512, 10, 640, 640))
    return HybridConfig(
        name="flashnext-moe", n_layers=48, hidden=2048, n_q_heads=16, n_kv_heads=2, head_dim=256,
        ffn_inter=512, vocab=151936, moe=MoEConfig(512, 10, 512, 512))


def scaled_hybrid(name: str = "hybrid-mini", n_layers: int = 4, hidden: int = 512, ffn: int = 1024,
                  vocab: int = 2048, q_heads: int = 6, kv_heads: int = 2, k_heads: int = 2,
                  v_heads: int = 6, drafter: bool = True, moe: Optional[MoEConfig] = None) -> HybridConfig:
    """A small model of the same architecture (tests, smoke)."""
    return HybridConfig(
        name=name, n_layers=n_layers, hidden=hidden, n_q_heads=q_heads, n_kv_heads=kv_heads,
        head_dim=256, ffn_inter=ffn, vocab=vocab, gdn_k_heads=k_heads, gdn_v_heads=v_heads,
        max_ctx=4096, moe=moe,
        drafter=DrafterConfig(hidden=hidden, n_layers=1, inter=ffn, block=4, n_taps=2) if drafter else None,
        w8_linears=("layers.0.mlp.down",))


@dataclass(frozen=True)
class TinyQwen3Config:
    """Plain Qwen3-style decoder used on CPU (fp32): plumbing and parity, no GPU."""
    n_layers: int = 2
    hidden: int = 256
    n_q_heads: int = 4
    n_kv_heads: int = 2
    head_dim: int = 64
    ffn_inter: int = 768
    vocab: int = 1024
    rope_theta: float = 1e6
    eps: float = 1e-6
    tie_embeddings: bool = True
    page_tokens: int = 16
    max_ctx: int = 4096
    name: str = "tiny-qwen3"


def by_name(name: str):
    table = {"qwen38-27b": qwen38_27b, "flashnext-moe": flashnext_moe,
             "flashnext-ref": lambda: flashnext_moe(True), "hybrid-mini": scaled_hybrid,
             "qwen38-27b-mxfp4": lambda: dataclasses.replace(qwen38_27b(), name="qwen38-27b-mxfp4", weight_format="mxfp4"),
             "qwen38-27b-nvfp4": lambda: dataclasses.replace(qwen38_27b(), name="qwen38-27b-nvfp4", weight_format="nvfp4"),
             "flashnext-moe-mxfp4": lambda: dataclasses.replace(flashnext_moe(), name="flashnext-moe-mxfp4",
                                                                moe=MoEConfig(512, 10, 512, 512, True, "mxfp4")),
             "qwen38-27b-dattn": lambda: dataclasses.replace(qwen38_27b(), name="qwen38-27b-dattn",
                                                             drafter=dataclasses.replace(qwen38_27b().drafter, attn_layers=1)),
             "tiny-qwen3": TinyQwen3Config}
    if name not in table:
        raise KeyError(f"unknown model {name!r}; known: {sorted(table)}")
    return table[name]()


def as_dict(cfg) -> dict:
    return dataclasses.asdict(cfg)
