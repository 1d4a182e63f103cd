"""The serving decode step of the flagship benchmark written with PyTorch + NCCL + library GEMMs only: the arm that
``bench.py`` measures the product against on the same box (the reference project itself cannot run on NVIDIA GPUs).

Same architecture, shapes, seeds and random streams as ``umdk_b200.models.dsv3_decoder.DecoderRank``:

* attention: torch gather of the selected KV rows through the block table, two batched matmuls and a softmax;
* KV offload: half of every sequence's pages in pinned host memory, ALL of them copied back every step with
  cudaMemcpyAsync (``Tensor.copy_(non_blocking=True)``) on a side stream, one contiguous copy per layer, ordered
  against the attention that reads them with events (the literal wording of the benchmark configuration);
* MoE: ``NcclLowLatencyMoe`` (all_gather dispatch, ONE grouped library GEMM per projection with no host
  synchronisation, reduce_scatter combine), the shared expert as one more group of the same grouped GEMM;
* everything else: the same torch ops as the product's decoder.
None of this package's kernels run here.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from umdk_b200.models.dsv3_decoder import DecoderConfig, build_dense_weights, expert_shard_stream
from umdk_b200.ops.ep_ll import ExpertWeights

from .nccl_baseline import GroupedFfn, NcclLowLatencyMoe

HEADS, DIM_V, KV_DIM, PAGE = 128, 512, 576, 64


def _cat8(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return torch.cat((a.view(torch.uint8), b.view(torch.uint8))).view(torch.float8_e4m3fn)


class BaselineDecoderRank:
    def __init__(self, cfg: DecoderConfig, group=None, device=None, gemm_backend: Optional[str] = None):
        self.cfg = c = cfg
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        dev = device or torch.device("cuda", torch.cuda.current_device())
        self.device = dev
        W = build_dense_weights(c, dev)
        self.embed, self.lm_head, self.final_norm, self.layers = W["embed"], W["lm_head"], W["final_norm"], W["layers"]
        backend = gemm_backend or GroupedFfn.pick_backend()
        self.gemm_backend = backend
        for L, (experts, shared) in zip(self.layers, expert_shard_stream(c, dev, self.rank, self.world, W["gen"])):
            if shared is not None:     # group 0 = the shared expert, groups 1.. = this rank's routed experts
                w = [_cat8(shared.w1q, experts.w1q), torch.cat((shared.w1s, experts.w1s)),
                     _cat8(shared.w2q, experts.w2q), torch.cat((shared.w2s, experts.w2s))]
            else:
                w = [experts.w1q, experts.w1s, experts.w2q, experts.w2s]
            del experts, shared
            ffn = GroupedFfn(*w, backend=backend, bmm_cap=self.world * c.batch)
            del w
            L["moe"] = NcclLowLatencyMoe(group, c.n_experts, c.top_k, ffn, shared_first=c.shared_expert)
        # KV cache laid out as the product's "pages" mode: resident pages, then a staging area for the offloaded half
        B, P = c.batch, c.ctx // PAGE
        half = P // 2
        self.n_resident, self.n_staging = B * (half + 1), B * half
        bt = torch.zeros(B, P + 1, dtype=torch.int64)
        for b in range(B):
            bt[b, :half] = torch.arange(half) + b * (half + 1)
            bt[b, P] = b * (half + 1) + half
            bt[b, half:P] = self.n_resident + b * half + torch.arange(half)
        self.block_table = bt.to(dev)
        self.new_row = (bt[:, P] * PAGE).to(dev)
        gk = torch.Generator(device=dev).manual_seed(c.seed + 5000 + self.rank)
        n_pages = self.n_resident + self.n_staging
        self.kv, self.host = [], []
        self.side = torch.cuda.Stream()
        for _ in range(c.n_layers):
            pool = torch.empty(n_pages, PAGE, KV_DIM, device=dev, dtype=torch.bfloat16)
            for s0 in range(0, n_pages, 4096):
                s1 = min(n_pages, s0 + 4096)
                pool[s0:s1] = (torch.randn(s1 - s0, PAGE, KV_DIM, device=dev, generator=gk) * 0.5).to(torch.bfloat16)
            self.kv.append(pool)
            if c.offload:
                h = torch.empty(self.n_staging, PAGE, KV_DIM, dtype=torch.bfloat16, pin_memory=True)
                h.copy_(pool[self.n_resident:])          # the state every decode step starts from
                self.host.append(h)
        self.ready = [torch.cuda.Event() for _ in range(c.n_layers)]
        self.consumed = [torch.cuda.Event() for _ in range(c.n_layers)]
        self._queued = False
        self.offload = c.offload
        pos = float(c.ctx)
        inv_freq = 1.0 / (c.rope_theta ** (torch.arange(0, c.qk_rope, 2, device=dev, dtype=torch.float32) / c.qk_rope))
        self.cos, self.sin = torch.cos(pos * inv_freq), torch.sin(pos * inv_freq)
        self.sm_scale = 1.0 / math.sqrt(c.qk_nope + c.qk_rope)
        self.h2d_bytes = 0
        torch.cuda.synchronize()

    def _rope(self, x):
        x1, x2 = x[..., 0::2].float(), x[..., 1::2].float()
        out = torch.stack((x1 * self.cos - x2 * self.sin, x1 * self.sin + x2 * self.cos), dim=-1)
        return out.flatten(-2).to(x.dtype)

    def prefetch(self):
        """Queues the copies that bring every offloaded page of every layer back, on the side stream; each waits for
        the attention that last read its staging area."""
        if not self.offload:
            return
        with torch.cuda.stream(self.side):
            for l in range(self.cfg.n_layers):
                self.side.wait_event(self.consumed[l])
                self.kv[l][self.n_resident:].copy_(self.host[l], non_blocking=True)
                self.ready[l].record(self.side)
                self.h2d_bytes += self.host[l].numel() * 2
        self._queued = True

    def _attention(self, l, q_full, indices):
        B = q_full.shape[0]
        idx = indices.to(torch.int64)
        page = torch.gather(self.block_table, 1, torch.div(idx, PAGE, rounding_mode="floor"))
        rows = self.kv[l].view(-1, KV_DIM)[page * PAGE + idx % PAGE]            # [B, topk, 576]
        s = torch.bmm(q_full, rows.transpose(1, 2)).float() * self.sm_scale   # [B, 128, topk]
        p = torch.softmax(s, dim=-1).to(torch.bfloat16)
        return torch.bmm(p, rows[..., :DIM_V])                                 # [B, 128, 512]

    def _layer(self, l, x, indices):
        c, L = self.cfg, self.layers[l]
        B, H = x.shape
        h = F.rms_norm(x, (H,), L["attn_norm"])
        qa = F.rms_norm(h @ L["wq_a"].t(), (c.q_lora,), L["q_norm"])
        q = (qa @ L["wq_b"].t()).view(B, HEADS, c.qk_nope + c.qk_rope)
        kva = h @ L["wkv_a"].t()
        ckv = F.rms_norm(kva[:, :DIM_V], (DIM_V,), L["kv_norm"])
        krope = self._rope(kva[:, DIM_V:])
        self.kv[l].view(-1, KV_DIM)[self.new_row] = torch.cat((ckv, krope), dim=-1)
        q_lat = torch.einsum("bhd,hdc->bhc", q[..., :c.qk_nope], L["w_uk"])
        q_full = torch.cat((q_lat, self._rope(q[..., c.qk_nope:])), dim=-1).contiguous()
        if self.offload:
            torch.cuda.current_stream().wait_event(self.ready[l])
        o_lat = self._attention(l, q_full, indices)
        if self.offload:
            self.consumed[l].record()
        o = torch.einsum("bhc,hcd->bhd", o_lat, L["w_uv"]).reshape(B, HEADS * c.v_head)
        x = x + o @ L["wo"].t()
        h = F.rms_norm(x, (H,), L["ffn_norm"])
        probs = torch.softmax((h @ L["router"].t()).float(), dim=-1)
        w, idx = torch.topk(probs, c.top_k, dim=-1)
        w = w / w.sum(dim=-1, keepdim=True)
        moe, share = L["moe"](h.contiguous(), idx, w)
        x = x + moe
        if share is not None:
            x = x + share
        return x

    def step(self, tokens: torch.Tensor, indices: List[torch.Tensor]) -> torch.Tensor:
        if self.offload and not self._queued:
            self.prefetch()
        self._queued = False
        x = self.embed[tokens]
        for l in range(self.cfg.n_layers):
            x = self._layer(l, x, indices[l])
        x = F.rms_norm(x, (self.cfg.hidden,), self.final_norm)
        return torch.argmax(x @ self.lm_head.t(), dim=-1)

    def wait_prefetch(self):
        if self.offload and self._queued:
            for l in range(self.cfg.n_layers):
                torch.cuda.current_stream().wait_event(self.ready[l])

    def close(self):
        self.kv, self.host, self.layers = [], [], []
