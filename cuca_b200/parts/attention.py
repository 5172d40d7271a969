"""Grouped-query attention over the paged cache.

q = h Wq^T, k = h Wk^T, v = h Wv^T (+ biases when the tensors exist); q and k
are rotated, k and v written to the request's pages, and each row attends to
keys lo..P of its request with scale 1/sqrt(head_dim) applied before the mask;
query head h reads key head h // (n_heads / n_kv_heads); then the output
projection is added to the stream (src/provider/local/model/cpu.rs:2822-2991,
3490-3521, model/cpu/paged_attn.rs:115-175, model/params.rs:704). The three
projections are stacked into one weight at load (the reference accepts the
stacked form: model/cpu.rs:3296-3301).

A layer that reads another layer's pages (`shares_cache`) has only q and o.
"""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from .base import POSITIONS, CacheNeeds, KvNeeds, Mixer, PartSpec, TensorNeed, register_mixer


@register_mixer("attention")
class PagedAttention(Mixer):
    """params: width, n_heads, n_kv_heads, head_dim, window (None: all keys), scale (None: 1/sqrt(head_dim)),
    position (PartSpec or None), shares_cache (bool). tensors: q, k, v, o and optional q_bias, k_bias,
    v_bias, o_bias."""

    graph_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.width = int(p["width"])
        self.n_heads = int(p["n_heads"])
        self.n_kv_heads = int(p["n_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.window = p.get("window")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.head_dim)
        self.shares_cache = bool(p.get("shares_cache", False))
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"{self.n_kv_heads} key heads must divide {self.n_heads} query heads")
        if not 1 <= self.head_dim <= ops.ATTENTION_MAX_HEAD_DIM:
            raise ValueError(f"attention: head size {self.head_dim} is outside what the kernels take "
                             f"(1..{ops.ATTENTION_MAX_HEAD_DIM})")
        pos = p.get("position")
        self.position = POSITIONS.get(pos.kind)(pos, runtime) if isinstance(pos, PartSpec) else None
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None

    # ------------------------------------------------------------ description
    def cache_needs(self):
        return CacheNeeds(kv=KvNeeds(self.n_kv_heads, self.head_dim, self.window))

    def tensors(self):
        t, d = self.spec.tensors, self.head_dim
        out = {t["q"]: TensorNeed((self.n_heads * d, self.width)),
               t["o"]: TensorNeed((self.width, self.n_heads * d))}
        if not self.shares_cache:
            out[t["k"]] = TensorNeed((self.n_kv_heads * d, self.width))
            out[t["v"]] = TensorNeed((self.n_kv_heads * d, self.width))
        for role, rows in (("q_bias", self.n_heads * d), ("k_bias", self.n_kv_heads * d),
                           ("v_bias", self.n_kv_heads * d), ("o_bias", self.width)):
            if role in t and not (self.shares_cache and role in ("k_bias", "v_bias")):
                out[t[role]] = TensorNeed((rows,), optional=True)
        return out

    def load(self, get):
        t = self.spec.tensors
        roles = ["q"] if self.shares_cache else ["q", "k", "v"]
        self.w_qkv = torch.cat([get(t[r]) for r in roles], dim=0).contiguous()
        biases = [get(t[r + "_bias"]) if r + "_bias" in t else None for r in roles]
        if any(b is not None for b in biases):
            if any(b is None for b in biases):
                raise ValueError("attention biases must be given for q, k and v together")
            self.b_qkv = torch.cat(biases).contiguous()
        self.w_o = get(t["o"])
        self.b_o = get(t["o_bias"]) if "o_bias" in t else None

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_qkv, self.w_o, self.b_qkv, self.b_o)
                   if w is not None)

    def prepare(self, context_length: int) -> None:
        if self.position is not None:
            self.position.prepare(context_length)

    # ------------------------------------------------------------ step
    def plan(self, step):
        """How this step's rows go to the attention kernels: made once per step from the per-request description
        (`StepBatch.req_row0/req_count/req_start`) and shared by the attention layers of the step."""
        return ops.attention_plan(step)

    def forward(self, h, stream, step, cache) -> None:
        stream = self.rt.stream(stream)
        nh, d = self.n_heads, self.head_dim
        nkv = 0 if self.shares_cache else self.n_kv_heads
        fused = self.position.fused_tables() if self.position is not None else None
        kpool, vpool = (None, None) if nkv == 0 else (cache.k, cache.v)
        plan = self.plan(step)
        if (fused is not None and self.rt.use_partials and h.shape[0] <= ops.ROPE_PARTIAL_MAX_ROWS
                and ops.gemm_partial_supported(h, self.w_qkv)):
            # few tokens: the projection leaves its K slices unadded; rotate-and-store adds them in 32-bit
            cos, sin, rot = fused
            parts = ops.gemm_partial(h, self.w_qkv, self.rt.err)
            if ops.attention_decode_fused_supported(plan, cache, h.dtype, h.shape[0], nh, self.n_kv_heads, d):
                # single tokens only: adding the slices, rotation, the page write and attention are one launch
                attn = self.rt.empty(h.shape[0], nh * d)
                chunk, n_splits = plan.chunk(self.n_kv_heads, d)
                ops.attention_decode_fused(parts, self.b_qkv, cos, sin, rot, nkv > 0, attn, cache.k, cache.v,
                                           step.positions, step.seq_of_row, cache.tables, None,
                                           plan.n_decode, nh, self.n_kv_heads, d, self.scale, self.window, chunk,
                                           n_splits, self.rt.err)
                stream.add_linear(attn, self.w_o, bias=self.b_o)
                return
            q = self.rt.empty(h.shape[0], nh * d)
            ops.rope_store_partial(parts, self.b_qkv, q, step.positions, step.seq_of_row, cache.tables, cos, sin, rot,
                                   kpool, vpool, cache.block_size, nh, nkv, d, self.rt.err)
        else:
            q = self.rt.linear(h, self.w_qkv, bias=self.b_qkv)  # [rows, (nh + 2 nkv) d]; q is the head of each row
            if fused is None:
                if self.position is not None:
                    self.position.apply(q, nh, nkv, d, step.positions)
                cos = sin = None
                rot = 0
            else:
                cos, sin, rot = fused
            ops.rope_store(q, step.positions, step.seq_of_row, cache.tables, cos, sin, rot, kpool, vpool,
                           cache.block_size, nh, nkv, d, self.rt.err)
        attn = self.rt.empty(h.shape[0], nh * d)
        ops.attention(q, attn, cache, step, plan, nh, self.n_kv_heads, d, self.scale, self.window, self.rt.err)
        stream.add_linear(attn, self.w_o, bias=self.b_o)
