"""fp32 torch reference of the decoder step (the checker for the floating-point path):
same ops, fp32 accumulation, bf16 rounding at the same points as the CUDA kernels.
Runs on CUDA when a GPU is there (full-size model), else on the CPU (small model)."""
import math

import numpy as np
import torch

from torq_b200.bf16 import from_bf16


def _bf(x):  # round an fp32 tensor to bf16 and back
    return x.to(torch.bfloat16).to(torch.float32)


class RefDecoder:
    def __init__(self, cfg, params, batch, device=None):
        self.cfg, self.B = cfg, batch
        self.dev = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(self.dev)
        f = lambda b: torch.from_numpy(from_bf16(b)).to(self.dev)
        self.embed_w, self.embed_s = t(params["embed"][0]), f(params["embed"][1])
        self.final_norm = f(params["final_norm"])
        self.layers = []
        for L in params["layers"]:
            d = {k: f(L[k]) for k in ("in_norm", "post_attn_norm", "pre_ffn_norm", "post_ffn_norm", "q_norm", "k_norm")}
            for k in ("qkv", "o", "gate_up", "down"):
                d[k] = (t(L[k][0]), f(L[k][1]))
            self.layers.append(d)
        D = cfg.head_dim
        self.kc = [torch.zeros(batch, cfg.max_seq, cfg.n_kv * D, device=self.dev) for _ in range(cfg.layers)]
        self.vc = [torch.zeros(batch, cfg.max_seq, cfg.n_kv * D, device=self.dev) for _ in range(cfg.layers)]
        self.mult = float(_bf(torch.tensor([math.sqrt(cfg.hidden)]))[0])
        self.trace = None  # set to a dict to record layer-0 intermediates of the next step

    def _norm(self, x, w, res=None):
        n = _bf(x * torch.rsqrt((x * x).mean(-1, keepdim=True) + self.cfg.eps) * (1.0 + w))
        return _bf(res + n) if res is not None else n

    @staticmethod
    def _gemv(x, ws):
        w, s = ws
        return _bf((x @ w.to(torch.float32).T) * s)

    def _gemv_chunked(self, x, ws, chunk=32768):
        w, s = ws
        outs = [(x @ w[i:i + chunk].to(torch.float32).T) * s[i:i + chunk] for i in range(0, w.shape[0], chunk)]
        return torch.cat(outs, -1)  # the LM head keeps fp32

    def step(self, tokens, pos):
        """tokens: int array [B]; returns (next token ids [B] int32, logits fp32 [B, V] holding bf16 values)."""
        cfg, B, D = self.cfg, self.B, self.cfg.head_dim
        tok = torch.as_tensor(np.asarray(tokens), device=self.dev).long()
        x = _bf(_bf(self.embed_w[tok].to(torch.float32) * self.embed_s[tok][:, None]) * self.mult)
        half = D // 2
        for li, L in enumerate(self.layers):
            glob = cfg.is_global(li)
            h = self._norm(x, L["in_norm"])
            qkv = self._gemv(h, L["qkv"])
            q = qkv[:, :cfg.n_q * D].reshape(B, cfg.n_q, D)
            k = qkv[:, cfg.n_q * D:(cfg.n_q + cfg.n_kv) * D].reshape(B, cfg.n_kv, D)
            v = qkv[:, (cfg.n_q + cfg.n_kv) * D:]
            q, k = self._norm(q, L["q_norm"]), self._norm(k, L["k_norm"])
            theta = cfg.theta_global if glob else cfg.theta_local
            inv = torch.pow(torch.tensor(theta, device=self.dev), -torch.arange(half, device=self.dev, dtype=torch.float32) / half)
            ang = pos * inv
            cs, sn = torch.cos(ang), torch.sin(ang)

            def rope(t):
                x1, x2 = t[..., :half], t[..., half:]
                return _bf(torch.cat([x1 * cs - x2 * sn, x2 * cs + x1 * sn], -1))
            q, k = rope(q), rope(k)
            self.kc[li][:, pos] = k.reshape(B, -1)
            self.vc[li][:, pos] = v
            lo = 0 if glob else max(0, pos - cfg.window + 1)
            K = self.kc[li][:, lo:pos + 1]                     # [B, T, D] (one KV head)
            V = self.vc[li][:, lo:pos + 1]
            s = torch.einsum("bhd,btd->bht", q * (D ** -0.5), K)
            p = torch.softmax(s, -1)
            a = _bf(torch.einsum("bht,btd->bhd", p, V)).reshape(B, -1)
            o = self._gemv(a, L["o"])
            if self.trace is not None and li == 0:
                self.trace.update(q=q.reshape(B, -1), a=a, o=o)
            x = self._norm(o, L["post_attn_norm"], res=x)
            h = self._norm(x, L["pre_ffn_norm"])
            gu = self._gemv(h, L["gate_up"])
            I = cfg.intermediate
            act = _bf(_bf(torch.nn.functional.gelu(gu[:, :I], approximate="tanh")) * gu[:, I:])
            d = self._gemv(act, L["down"])
            if self.trace is not None and li == 0:
                self.trace.update(x1=x, h2=h, gu=gu, act=act, d=d)
            x = self._norm(d, L["post_ffn_norm"], res=x)
            if self.trace is not None and li == 0:
                self.trace.update(x2=x)
            if self.trace is not None:
                self.trace['layer%d' % li] = x
                self.trace['attn%d' % li] = a
                self.trace['q%d' % li] = q.reshape(B, -1)
        x = self._norm(x, self.final_norm)
        if self.trace is not None:
            self.trace['final'] = x
        logits = self._gemv_chunked(x, (self.embed_w, self.embed_s))
        return logits.argmax(-1).to(torch.int32).cpu().numpy(), logits.cpu().numpy()
