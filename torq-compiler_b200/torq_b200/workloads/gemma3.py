"""Gemma-3-1B-architecture decoder step, random-init, int8 per-output-channel symmetric
weights with bf16 scales, bf16 activations and KV cache, as an op-list graph.

Shape (full size): 26 layers, hidden 1152, 4 query heads and 1 KV head of 256 dims, GeGLU
MLP with intermediate 6912, vocabulary 262144 with the embedding tied to the LM head,
RMSNorm before and after attention and MLP plus per-head q/k norms, RoPE theta 10k on
local layers (sliding window 512) and 1M on global layers, 5 local layers to 1 global.

One executable = one decode step for a fixed batch: inputs are the current token ids [B]
and the position [1] (the same for the whole batch); outputs the greedy next token ids
[B] (and the logits when `with_logits`). The KV caches are state tensors that persist
across dispatches; a prompt is consumed by running the same step once per prompt token.

Weights are uniform int8 in [-127, 127] with scales 1 / (127 * sqrt(K)) * g so that
activations stay O(1); values stand in for a checkpoint, nothing is loaded.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

from ..bf16 import from_bf16, to_bf16
from ..oplist import Graph


@dataclass
class GemmaConfig:
    layers: int = 26
    hidden: int = 1152
    n_q: int = 4
    n_kv: int = 1
    head_dim: int = 256
    intermediate: int = 6912
    vocab: int = 262144
    window: int = 512
    local_per_global: int = 5
    theta_local: float = 10000.0
    theta_global: float = 1000000.0
    eps: float = 1e-6
    max_seq: int = 1152

    def is_global(self, layer: int) -> bool:
        return (layer + 1) % (self.local_per_global + 1) == 0


SMALL = GemmaConfig(layers=3, hidden=256, intermediate=512, vocab=4096, window=24, local_per_global=2, max_seq=96)


def _weight(rng, n, k, gain=1.0):
    w = rng.integers(-127, 128, (n, k), dtype=np.int8)
    scale = (gain / (127.0 / math.sqrt(3.0) * math.sqrt(k))) * rng.uniform(0.8, 1.25, n)
    return w, to_bf16(scale.astype(np.float32))


def _norm_w(rng, n, mean=0.0):
    return to_bf16(rng.normal(mean, 0.1 if mean == 0.0 else 0.03, n).astype(np.float32))


def random_weights(cfg: GemmaConfig, seed: int = 1234, embed_gain: float = 0.02) -> dict:
    """All parameters as numpy arrays (shared by the graph builder and the reference model).
    embed_gain sets how strongly the tied embedding shows in the residual stream: 0.02 gives the
    nearly flat logits of an untrained model, ~0.3 gives peaked logits (the input token wins)."""
    rng = np.random.default_rng(seed)
    H, D = cfg.hidden, cfg.head_dim
    # a small embedding gain (x0 has RMS ~ 0.7 after the sqrt(H) normaliser) keeps the tied token
    # embedding from dominating the residual stream; otherwise a random-init model repeats its input
    P = {"embed": _weight(rng, cfg.vocab, H, gain=embed_gain), "final_norm": _norm_w(rng, H), "layers": []}
    for _ in range(cfg.layers):
        P["layers"].append(dict(
            # post-sublayer norms scale their branch to about a quarter of unit RMS (1 + w ~ 0.25),
            # as trained checkpoints do: the residual stream then changes gradually from layer to
            # layer instead of being re-randomised by every branch
            in_norm=_norm_w(rng, H), post_attn_norm=_norm_w(rng, H, -0.75), pre_ffn_norm=_norm_w(rng, H),
            post_ffn_norm=_norm_w(rng, H, -0.75), q_norm=_norm_w(rng, D), k_norm=_norm_w(rng, D),
            qkv=_weight(rng, (cfg.n_q + 2 * cfg.n_kv) * D, H), o=_weight(rng, H, cfg.n_q * D),
            gate_up=_weight(rng, 2 * cfg.intermediate, H, gain=1.5), down=_weight(rng, H, cfg.intermediate)))
    return P


def shard_weights(cfg: GemmaConfig, params: dict, tp: int, rank: int) -> dict:
    """Megatron-style shard `rank` of `tp` (tensor parallelism over the GPUs of one node):
    q heads and the gate/up rows are split by output row, the o and down projections by input
    column (their partial results are summed across the GPUs), the LM head by vocabulary row;
    the single KV head, the norms and the embedding table are replicated."""
    if cfg.n_kv != 1 or cfg.n_q % tp or cfg.intermediate % tp or cfg.vocab % tp:
        raise ValueError("the group size must divide the query heads, the MLP width and the vocabulary")
    D, I = cfg.head_dim, cfg.intermediate
    hq, Il, Vl = cfg.n_q // tp, I // tp, cfg.vocab // tp
    q_rows = np.arange(rank * hq * D, (rank + 1) * hq * D)
    kv_rows = np.arange(cfg.n_q * D, (cfg.n_q + 2) * D)
    gu_rows = np.concatenate([np.arange(rank * Il, (rank + 1) * Il), I + np.arange(rank * Il, (rank + 1) * Il)])
    out = {"embed": params["embed"], "final_norm": params["final_norm"], "layers": [],
           "lm_head": (np.ascontiguousarray(params["embed"][0][rank * Vl:(rank + 1) * Vl]),
                       np.ascontiguousarray(params["embed"][1][rank * Vl:(rank + 1) * Vl])),
           "vocab_offset": rank * Vl}
    for L in params["layers"]:
        rows = np.concatenate([q_rows, kv_rows])
        S = dict(L)
        S["qkv"] = (np.ascontiguousarray(L["qkv"][0][rows]), np.ascontiguousarray(L["qkv"][1][rows]))
        S["o"] = (np.ascontiguousarray(L["o"][0][:, rank * hq * D:(rank + 1) * hq * D]), L["o"][1])
        S["gate_up"] = (np.ascontiguousarray(L["gate_up"][0][gu_rows]), np.ascontiguousarray(L["gate_up"][1][gu_rows]))
        S["down"] = (np.ascontiguousarray(L["down"][0][:, rank * Il:(rank + 1) * Il]), L["down"][1])
        out["layers"].append(S)
    return out


def build_decode_step(cfg: GemmaConfig, batch: int, params: dict, with_logits: bool = False, tp: int = 1,
                      rank: int = 0) -> Graph:
    """tp > 1: `params` is shard_weights(cfg, full_params, tp, rank); the graph is that GPU's share
    of the step (logits, when asked for, are the shard's [B, vocab / tp] slice)."""
    g = Graph()
    H, D = cfg.hidden, cfg.head_dim
    n_q = cfg.n_q // tp
    tokens = g.input((batch,), "i32")
    pos = g.input((1,), "i32")
    table = g.const(params["embed"][0])
    table_scale = g.const(params["embed"][1], "bf16")
    mult = float(from_bf16(to_bf16(np.array([math.sqrt(H)], np.float32)))[0])  # the normaliser is a bf16 value
    x = g.embed(tokens, table, table_scale, mult)
    for li, L in enumerate(params["layers"]):
        glob = cfg.is_global(li)
        kc = g.state((batch, cfg.max_seq, cfg.n_kv * D), "bf16")
        vc = g.state((batch, cfg.max_seq, cfg.n_kv * D), "bf16")
        h = g.rmsnorm(x, L["in_norm"], cfg.eps)
        qkv = g.gemv_w8(h, *L["qkv"])
        q = g.rope_kv(qkv, pos, L["q_norm"], L["k_norm"], kc, vc, n_q=n_q, n_kv=cfg.n_kv, head_dim=D,
                      theta=cfg.theta_global if glob else cfg.theta_local, eps=cfg.eps)
        a = g.attn_decode(q, pos, kc, vc, n_q=n_q, n_kv=cfg.n_kv, head_dim=D, window=0 if glob else cfg.window,
                          scale=D ** -0.5)
        o = g.gemv_w8(a, *L["o"]) if tp == 1 else g.allreduce(g.gemv_w8(a, *L["o"], out_dtype="f32"), tp, rank)
        x = g.rmsnorm(o, L["post_attn_norm"], cfg.eps, residual=x)
        h = g.rmsnorm(x, L["pre_ffn_norm"], cfg.eps)
        gu = g.gemv_w8(h, *L["gate_up"])
        act = g.geglu(gu)
        d = g.gemv_w8(act, *L["down"]) if tp == 1 else g.allreduce(g.gemv_w8(act, *L["down"], out_dtype="f32"), tp, rank)
        x = g.rmsnorm(d, L["post_ffn_norm"], cfg.eps, residual=x)
    x = g.rmsnorm(x, params["final_norm"], cfg.eps)
    if tp == 1:
        logits = g.gemv_w8(x, table, table_scale, out_dtype="f32")  # logits stay fp32: greedy ids do not hinge on bf16 ties
        nxt = g.argmax(logits)
    else:
        logits = g.gemv_w8(x, *params["lm_head"], out_dtype="f32")
        nxt = g.argmax(logits, vocab_offset=params["vocab_offset"], group_size=tp)
    g.output(nxt)
    if with_logits:
        g.output(logits)
    return g


def weight_bytes_per_token(cfg: GemmaConfig) -> int:
    """int8 weight bytes one decode step streams (the algorithmic bytes of the step)."""
    H, D, I = cfg.hidden, cfg.head_dim, cfg.intermediate
    per_layer = (cfg.n_q + 2 * cfg.n_kv) * D * H + H * cfg.n_q * D + 2 * I * H + H * I
    return cfg.layers * per_layer + cfg.vocab * H
