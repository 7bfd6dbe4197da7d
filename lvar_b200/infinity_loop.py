"""Random-init generation loop with the Infinity-2B architecture, the caller of the sparse-attention path.

This restates, for benchmarking, what surrounds the path during text-to-image generation in
``SparVAR_Infinity.autoregressive_infer_cfg`` (models/sparvar/sparvar_model.py:488-721) with blocks shaped like
``CrossAttnBlock`` (models/sparvar/basic_sparvar.py:396-468): 13 scales x ``depth`` blocks, a conditional and
an unconditional copy of every prompt (classifier-free guidance on the logits), a KV cache over all scales,
bit-label sampling and the multi-scale code accumulation that produces the next scale's input.

Every SELF-attention call goes through this package: the fused QKV prologue (L2-normalise, per-head scale,
2-D RoPE, append to the bf16 KV cache) and :class:`lvar_b200.policy.SelfAttentionDispatch` (dense attention
below the decision scale, CS4A in the first layers and CSLA in the remaining ones from it on).  Everything
off that path is plain PyTorch: linear layers (cuBLAS), layer norms, GELU, the 64-token cross-attention
(``scaled_dot_product_attention``), sampling and interpolation.  Weights are random (there is no checkpoint to
load); the image decoder is not part of the loop.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from . import kernels as K
from . import policy as P
from .sparse_attn_config import GLOBAL_CONFIG


@dataclass
class LoopConfig:
    depth: int = 32
    width: int = 2048
    heads: int = 16
    ffn: int = 8192
    text_dim: int = 2048
    text_len: int = 64
    code_dim: int = 32                      # bits per token of the bitwise tokenizer
    scales: Sequence[int] = field(default_factory=lambda: tuple(P.INFINITY_SCALES))
    cfg: float = 3.0                        # guidance strength on the logits
    tau: float = 1.0
    # "sparse": the per-(scale, layer) dispatch; "dense": dense self-attention everywhere (the baseline model);
    # "none": the prologue still runs but no attention does (o = q) - for measuring self-attention's share
    attn_mode: str = "sparse"

    @property
    def head_dim(self) -> int:
        return self.width // self.heads


def rope2d_tables(scales: Sequence[int], head_dim: int, base: float = 10000.0, device="cpu"):
    """cos/sin fp32 [sum(s*s), head_dim/2], one row per token of the multi-scale sequence: a token at (y, x) of
    an s x s map is given the position of the nearest point of the LAST scale's grid; the first half of a row
    rotates by the y position, the second half by the x position (models/infinity/basic_infinity.py:42-133 with
    rope2d_normalized_by_hw = 2)."""
    half = head_dim // 2
    quarter = half // 2
    theta = base ** (-torch.arange(quarter, dtype=torch.float32) * 2.0 / half)
    last = scales[-1]
    out = []
    for s in scales:
        pos = torch.round(torch.arange(s, dtype=torch.float32) * (last / s))
        ang = pos.view(-1, 1) * theta.view(1, -1)                              # [s, quarter]
        row = torch.cat([ang.view(s, 1, quarter).expand(s, s, quarter),         # y
                         ang.view(1, s, quarter).expand(s, s, quarter)], -1)    # x
        out.append(row.reshape(s * s, half))
    ang = torch.cat(out, 0).to(device)
    return torch.cos(ang).contiguous(), torch.sin(ang).contiguous()


class _Block:
    """Weights of one transformer block (bf16 matrices, fp32 modulation vectors)."""

    def __init__(self, cfg: LoopConfig, gen: torch.Generator, device):
        C, Fh, T = cfg.width, cfg.ffn, cfg.text_dim

        def w(o, i):
            return (torch.randn(o, i, generator=gen, device=device, dtype=torch.float32) * (i ** -0.5)).bfloat16()

        def b(n):
            return torch.zeros(n, device=device, dtype=torch.bfloat16)
        self.w_qkv, self.b_qkv = w(3 * C, C), b(3 * C)
        self.scale_mul = torch.full((cfg.heads,), 4.0, device=device, dtype=torch.float32)
        self.w_proj, self.b_proj = w(C, C), b(C)
        self.ca_norm_w = torch.ones(C, device=device)
        self.ca_norm_b = torch.zeros(C, device=device)
        self.w_caq, self.b_caq = w(C, C), b(C)
        self.w_cakv, self.b_cakv = w(2 * C, T), b(2 * C)
        self.w_caproj, self.b_caproj = w(C, C), b(C)
        self.ca_gamma = torch.full((C,), 0.1, device=device)
        self.w_fc1, self.b_fc1 = w(Fh, C), b(Fh)
        self.w_fc2, self.b_fc2 = w(C, Fh), b(C)
        self.ada = torch.randn(6, C, generator=gen, device=device) * (C ** -0.5)


class InfinityLoop:
    """``generate(text)``: text bf16 [B, text_len, text_dim] -> accumulated codes fp32 [B, code_dim, S, S]
    (S = the last scale's side).  One instance holds the weights, the KV caches of every layer (bf16
    [2B, heads, total tokens, head_dim]) and the per-layer attention state for a fixed batch size."""

    def __init__(self, cfg: LoopConfig, batch: int, device="cuda", seed: int = 0):
        self.cfg, self.B, self.device = cfg, batch, torch.device(device)
        gen = torch.Generator(device=self.device).manual_seed(seed)
        C, c, Hn = cfg.width, cfg.head_dim, cfg.heads
        self.cum = P.cumulative_tokens(cfg.scales)
        self.blocks = [_Block(cfg, gen, self.device) for _ in range(cfg.depth)]

        def w(o, i):
            return (torch.randn(o, i, generator=gen, device=self.device) * (i ** -0.5)).bfloat16()
        self.w_text, self.w_text2 = w(C, cfg.text_dim), w(cfg.text_dim, C)        # text tokens for cross-attention
        self.w_sos = w(C, cfg.text_dim)                                          # pooled text -> first token / condition
        self.w_ada = (torch.randn(6 * C, C, generator=gen, device=self.device) * (C ** -0.5) * 0.1)
        self.uncond = torch.randn(cfg.text_len, cfg.text_dim, generator=gen, device=self.device).bfloat16()
        self.pos_start = torch.randn(1, 1, C, generator=gen, device=self.device) * 0.02
        self.lvl_embed = torch.randn(len(cfg.scales), C, generator=gen, device=self.device) * 0.02
        self.w_embed, self.b_embed = w(C, cfg.code_dim), torch.zeros(C, device=self.device, dtype=torch.bfloat16)
        self.w_head_ada = torch.randn(2 * C, C, generator=gen, device=self.device) * (C ** -0.5) * 0.1
        self.w_head = torch.randn(2 * cfg.code_dim, C, generator=gen, device=self.device) * (C ** -0.5)
        self.rope_cos, self.rope_sin = rope2d_tables(cfg.scales, c, device=self.device)
        bs = 2 * batch
        self.k_cache = [torch.zeros(bs, Hn, self.cum[-1], c, device=self.device, dtype=torch.bfloat16)
                        for _ in range(cfg.depth)]
        self.v_cache = [torch.zeros_like(t) for t in self.k_cache]
        attn_cfg = GLOBAL_CONFIG["attn"]
        self.dispatch = [P.SelfAttentionDispatch(i, attn_cfg, cfg.scales, scale=1.0) for i in range(cfg.depth)]
        if cfg.attn_mode not in ("sparse", "dense", "none"):
            raise ValueError(f"attn_mode must be 'sparse', 'dense' or 'none', got {cfg.attn_mode!r}")
        self.csla = (P.build_csla_list(cfg.scales, attn_cfg, Hn, device=self.device) if cfg.attn_mode == "sparse"
                     else [None] * len(cfg.scales))
        self.routes: Dict[str, int] = {}
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._static: Dict[str, torch.Tensor] = {}

    # -- one block ---------------------------------------------------------------------------------
    def _self_attention(self, blk: _Block, li: int, xn: torch.Tensor, si: int) -> torch.Tensor:
        cfg = self.cfg
        bs, L, C = xn.shape
        qkv = F.linear(xn, blk.w_qkv, blk.b_qkv).view(bs, L, 3, cfg.heads, cfg.head_dim)
        pos = self.cum[si]
        q = K.qkv_prologue(qkv, blk.scale_mul, self.rope_cos, self.rope_sin, pos, self.k_cache[li], self.v_cache[li], pos)
        k = self.k_cache[li][:, :, :self.cum[si + 1]]
        v = self.v_cache[li][:, :, :self.cum[si + 1]]
        d = self.dispatch[li]
        if cfg.attn_mode == "sparse":
            o = d(q, k, v, scale_ind=si, layer_ind=li, spattn_fn=self.csla[si])
        elif cfg.attn_mode == "dense":
            o = K.dense_attn_fwd(q, k, v, 1.0, return_stats=False)[0]
            d.last_route = "dense"
        else:
            o = q
            d.last_route = "none"
        self.routes[d.last_route] = self.routes.get(d.last_route, 0) + 1
        return F.linear(o.transpose(1, 2).reshape(bs, L, C), blk.w_proj, blk.b_proj)

    def _cross_attention(self, blk: _Block, x: torch.Tensor, text_kv) -> torch.Tensor:
        cfg = self.cfg
        bs, L, C = x.shape
        xn = F.layer_norm(x, (C,), blk.ca_norm_w, blk.ca_norm_b, 1e-6).bfloat16()
        q = F.linear(xn, blk.w_caq, blk.b_caq).view(bs, L, cfg.heads, cfg.head_dim).transpose(1, 2)
        tk, tv = text_kv
        o = F.scaled_dot_product_attention(q, tk, tv)
        return F.linear(o.transpose(1, 2).reshape(bs, L, C), blk.w_caproj, blk.b_caproj)

    def _block(self, li: int, x: torch.Tensor, mod: torch.Tensor, text_kv, si: int) -> torch.Tensor:
        """x fp32 [2B, L, C]; mod fp32 [2B, 6, C] (the condition's six modulation vectors)."""
        blk = self.blocks[li]
        C = x.shape[-1]
        g1, g2, s1, s2, h1, h2 = (blk.ada.unsqueeze(0) + mod).unsqueeze(2).unbind(1)   # each [2B, 1, C]
        xn = (F.layer_norm(x, (C,), None, None, 1e-6) * (s1 + 1) + h1).bfloat16()
        x = x + self._self_attention(blk, li, xn, si).float() * g1
        x = x + self._cross_attention(blk, x, text_kv).float() * blk.ca_gamma
        xn = (F.layer_norm(x, (C,), None, None, 1e-6) * (s2 + 1) + h2).bfloat16()
        hid = F.gelu(F.linear(xn, blk.w_fc1, blk.b_fc1), approximate="tanh")
        return x + F.linear(hid, blk.w_fc2, blk.b_fc2).float() * g2

    # -- the loop ----------------------------------------------------------------------------------
    def _text_kv(self, text2: torch.Tensor) -> List:
        """Per block: projected text keys / values [2B, heads, text_len, head_dim]."""
        cfg = self.cfg
        bs, T, _ = text2.shape
        t = F.linear(torch.tanh(F.linear(text2, self.w_text)), self.w_text2)
        out = []
        for blk in self.blocks:
            kv = F.linear(t, blk.w_cakv, blk.b_cakv).view(bs, T, 2, cfg.heads, cfg.head_dim)
            out.append((kv[:, :, 0].transpose(1, 2), kv[:, :, 1].transpose(1, 2)))
        return out

    def _generate(self, text: torch.Tensor, noise: List[torch.Tensor]) -> torch.Tensor:
        cfg, B = self.cfg, self.B
        C, S = cfg.width, cfg.scales[-1]
        text2 = torch.cat([text, self.uncond.unsqueeze(0).expand_as(text)], 0)            # conditional | unconditional
        pooled = F.linear(text2.mean(1), self.w_sos).float()                              # [2B, C]
        mod = F.linear(F.silu(pooled), self.w_ada).view(2 * B, 6, C)
        head_mod = F.linear(F.silu(pooled), self.w_head_ada).view(2 * B, 1, 2, C)
        text_kv = self._text_kv(text2)
        x = pooled.unsqueeze(1) + self.pos_start
        summed = torch.zeros(B, cfg.code_dim, S, S, device=self.device)
        for si, side in enumerate(cfg.scales):
            x = x + self.lvl_embed[si]
            for li in range(cfg.depth):
                x = self._block(li, x, mod, text_kv[li], si)
            hn = F.layer_norm(x, (C,), None, None, 1e-6) * (head_mod[:, :, 0] + 1) + head_mod[:, :, 1]
            logits = F.linear(hn, self.w_head) * (1.0 / cfg.tau)                         # [2B, L, 2*code_dim]
            logits = cfg.cfg * logits[:B] + (1.0 - cfg.cfg) * logits[B:]
            two = logits.view(B, side * side, cfg.code_dim, 2)
            bit = noise[si] < torch.sigmoid(two[..., 1] - two[..., 0])                   # a draw from softmax over 2 classes
            codes = (bit.float() * 2.0 - 1.0) * (cfg.code_dim ** -0.5)
            codes = codes.view(B, side, side, cfg.code_dim).permute(0, 3, 1, 2)
            if si + 1 < len(cfg.scales):
                summed = summed + F.interpolate(codes, size=(S, S), mode="bilinear", align_corners=False)
                nxt = cfg.scales[si + 1]
                inp = F.interpolate(summed, size=(nxt, nxt), mode="bilinear", align_corners=False)
                inp = inp.flatten(2).transpose(1, 2).bfloat16()                          # [B, L', code_dim]
                x = F.linear(inp, self.w_embed, self.b_embed).float().repeat(2, 1, 1)
            else:
                summed = summed + codes
        return summed

    def make_noise(self, seed: int = 0) -> List[torch.Tensor]:
        """The sampler's uniform draws, one tensor per scale (drawn up front so that the loop itself is free of
        random-number state and can be replayed as a CUDA graph)."""
        gen = torch.Generator(device=self.device).manual_seed(seed)
        return [torch.rand(self.B, s * s, self.cfg.code_dim, generator=gen, device=self.device)
                for s in self.cfg.scales]

    def generate(self, text: torch.Tensor, seed: int = 0) -> torch.Tensor:
        """Eager generation of one batch."""
        assert text.shape == (self.B, self.cfg.text_len, self.cfg.text_dim) and text.dtype == torch.bfloat16
        self.routes = {}
        return self._generate(text, self.make_noise(seed))

    def capture(self, text: torch.Tensor, seed: int = 0) -> None:
        """Captures one whole generation (all scales and blocks) in a CUDA graph on a side stream, after a warm-up
        run on that stream that creates the per-layer tables and scratch.  ``replay`` then regenerates from the
        current contents of the static text and noise buffers."""
        self._static = {"text": text.clone(), "noise": self.make_noise(seed)}
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            self.routes = {}
            self._generate(self._static["text"], self._static["noise"])
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph, stream=side):
            self._static["out"] = self._generate(self._static["text"], self._static["noise"])

    def replay(self, text: Optional[torch.Tensor] = None) -> torch.Tensor:
        assert self._graph is not None, "call capture() first"
        if text is not None:
            self._static["text"].copy_(text)
        self._graph.replay()
        return self._static["out"]

    def flops_per_batch(self) -> Dict[str, float]:
        """Algorithmic FLOPs of one generation of this instance's batch: linear layers (2*m*n*k) and dense
        self-attention (4*D*Lq*Lkv per head) summed over scales, blocks and the 2B sequences."""
        cfg = self.cfg
        C, Fh, T = cfg.width, cfg.ffn, cfg.text_dim
        per_token = 2.0 * (3 * C * C + C * C + C * C + C * C + 2 * C * Fh)      # qkv, proj, ca q, ca proj, ffn
        tokens = self.cum[-1]
        lin = cfg.depth * 2 * self.B * tokens * per_token
        attn = sum(4.0 * cfg.head_dim * (s * s) * self.cum[i + 1] for i, s in enumerate(cfg.scales))
        attn *= cfg.depth * 2 * self.B * cfg.heads
        return {"linear": lin, "self_attention_dense": attn}
