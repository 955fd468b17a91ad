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


def shard_layout(cfg: GemmaConfig, tp: int, rank: int) -> dict:
    """Which rows and columns rank `rank` of `tp` owns. Up to n_q GPUs each take whole query heads; beyond
    that (tp a multiple of n_q) a head is computed by tp / n_q GPUs, each of which takes a column slice of
    that head for the o projection. The MLP width is split in blocks of 64 (unevenly when it must be)."""
    D, I, nq = cfg.head_dim, cfg.intermediate, cfg.n_q
    if cfg.n_kv != 1 or I % 64 or cfg.vocab % tp or not (nq % tp == 0 or tp % nq == 0) or (nq * D // tp) % 64:
        raise ValueError("unsupported tensor-parallel group size for this shape")
    share = max(1, tp // nq)            # GPUs per head
    hq = max(1, nq // tp)               # heads per GPU
    head0 = rank // share if tp > nq else rank * hq
    o_k = nq * D // tp
    nb, base, extra = I // 64, (I // 64) // tp, (I // 64) % tp
    i0 = 64 * (rank * base + min(rank, extra))
    i1 = i0 + 64 * (base + (1 if rank < extra else 0))
    return dict(heads=hq, head0=head0, o_cols=(rank * o_k, (rank + 1) * o_k), o_k_offset=rank * o_k - head0 * D,
                mlp=(i0, i1), vocab=(rank * cfg.vocab // tp, (rank + 1) * cfg.vocab // tp))


def shard_weights(cfg: GemmaConfig, params: dict, tp: int, rank: int) -> dict:
    """Megatron-style shard `rank` of `tp` (tensor parallelism over the GPUs of one node):
    q heads and the gate/up rows are split by output row, the o and down projections by input
    column (their partial results are summed across the GPUs), the LM head by vocabulary row;
    the single KV head, the norms and the embedding table are replicated."""
    lay = shard_layout(cfg, tp, rank)
    D, I = cfg.head_dim, cfg.intermediate
    q_rows = np.arange(lay["head0"] * D, (lay["head0"] + lay["heads"]) * D)
    kv_rows = np.arange(cfg.n_q * D, (cfg.n_q + 2) * D)
    i0, i1 = lay["mlp"]
    gu_rows = np.concatenate([np.arange(i0, i1), I + np.arange(i0, i1)])
    v0, v1 = lay["vocab"]
    out = {"embed": params["embed"], "final_norm": params["final_norm"], "layers": [],
           "lm_head": (np.ascontiguousarray(params["embed"][0][v0:v1]), np.ascontiguousarray(params["embed"][1][v0:v1])),
           "vocab_offset": v0, "layout": lay}
    for L in params["layers"]:
        rows = np.concatenate([q_rows, kv_rows])
        S = dict(L)
        S["qkv"] = (np.ascontiguousarray(L["qkv"][0][rows]), np.ascontiguousarray(L["qkv"][1][rows]))
        S["o"] = (np.ascontiguousarray(L["o"][0][:, lay["o_cols"][0]:lay["o_cols"][1]]), L["o"][1])
        S["gate_up"] = (np.ascontiguousarray(L["gate_up"][0][gu_rows]), np.ascontiguousarray(L["gate_up"][1][gu_rows]))
        S["down"] = (np.ascontiguousarray(L["down"][0][:, i0:i1]), L["down"][1])
        out["layers"].append(S)
    return out


def build_decode_step(cfg: GemmaConfig, batch: int, params: dict, with_logits: bool = False, tp: int = 1,
                      rank: int = 0) -> Graph:
    """tp > 1: `params` is shard_weights(cfg, full_params, tp, rank); the graph is that GPU's share
    of the step (logits, when asked for, are the shard's [B, vocab / tp] slice)."""
    g = Graph()
    H, D = cfg.hidden, cfg.head_dim
    n_q = params["layout"]["heads"] if tp > 1 else cfg.n_q
    o_k_offset = params["layout"]["o_k_offset"] if tp > 1 else 0
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
        o = g.gemv_w8(a, *L["o"]) if tp == 1 else g.allreduce(g.gemv_w8(a, *L["o"], out_dtype="f32", in_offset=o_k_offset), tp, rank)
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
