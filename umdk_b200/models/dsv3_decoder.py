"""DeepSeek-V3-shaped MoE decoder for the serving decode step (one token per sequence per step).

Per layer: RMSNorm -> multi-head latent attention with absorbed projections, computed by the sparse top-k MLA
flash-decode kernel over a paged KV cache whose second half of pages lives in pinned host memory and is prefetched
on a side stream -> RMSNorm -> softmax top-k router -> expert-parallel low-latency MoE (fp8 dispatch, tcgen05 grouped
GEMMs, combine fused in the down-projection epilogue) plus a shared expert. Attention is data parallel (every rank
decodes its own batch), experts are sharded over the ranks of the EP group.

Dense projections (q/kv/o, router, lm_head) are plain library GEMMs through torch.matmul; everything between them
(residual adds, RMSNorm, rotary embedding, the KV row write, the router's softmax / top-k / renormalisation) runs in
the fused kernels of ops/glue.py, and the step is replayed as CUDA graphs: one graph per stretch between two
attention calls (the attention launches and the event waits of the KV prefetch stay outside the graphs). The
reference project has no model code; the architecture and shapes come from the serving benchmark configuration.
``DecoderRank.step_eager`` is the same step written with plain torch ops (the oracle of the fused path).
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .. import _native
from ..ops import glue
from ..ops import reference as ref
from ..ops.attention import DIM as KV_DIM, DIM_V, HEADS, PAGE, sparse_mla_decode
from ..ops.ep_ll import EpLowLatency, ExpertWeights
from ..ops.kv_offload import KvOffloadManager
from ..parallel.symm import SymmetricHeap


@dataclass
class DecoderConfig:
    hidden: int = 7168
    n_layers: int = 4
    q_lora: int = 1536
    qk_nope: int = 128
    qk_rope: int = 64
    v_head: int = 128
    n_experts: int = 256
    top_k: int = 8
    moe_ffn: int = 2048
    shared_expert: bool = True
    vocab: int = 129280
    batch: int = 64          # sequences per rank
    ctx: int = 32768         # tokens already in the cache
    topk_kv: int = 2048      # KV rows attended per query
    offload: bool = True     # second half of each sequence's pages in pinned host memory
    # how offloaded KV comes back each step: "rows" = gather only the token rows the step's top-k indices select
    # (zero-copy reads of the pinned pool by a kernel on the side stream); "pages" = cudaMemcpyAsync of every
    # offloaded page into a device staging area as large as the offloaded half
    kv_fetch: str = "rows"
    rope_theta: float = 10000.0
    seed: int = 0

    @staticmethod
    def tiny() -> "DecoderConfig":
        return DecoderConfig(hidden=1024, n_layers=2, q_lora=256, n_experts=16, top_k=4, moe_ffn=256, vocab=2048,
                             batch=8, ctx=1024, topk_kv=256)


def _quant_experts(n: int, rows: int, cols: int, gen_device, gen: torch.Generator, std: float = 0.02):
    """n expert matrices [rows, cols] drawn N(0, std) in bf16, quantised to fp8 e4m3 with 128x128 block scales."""
    q = torch.empty(n, rows, cols, dtype=torch.uint8, device=gen_device).view(torch.float8_e4m3fn)
    s = torch.empty(n, rows // 128, cols // 128, dtype=torch.float32, device=gen_device)
    for i in range(n):
        w = torch.randn(rows, cols, device=gen_device, generator=gen, dtype=torch.float32) * std
        wf = w.reshape(rows // 128, 128, cols // 128, 128)
        amax = wf.abs().amax(dim=(1, 3)).clamp_min(1e-4)
        q[i] = (wf * (448.0 / amax)[:, None, :, None]).reshape(rows, cols).to(torch.float8_e4m3fn)
        s[i] = amax / 448.0
    return q, s


def build_dense_weights(cfg: DecoderConfig, dev) -> dict:
    """Replicated (non-expert) weights of the decoder, N(0, 0.02) in bf16, the same on every rank (seed ``cfg.seed``).
    Returns {"embed", "lm_head", "final_norm", "layers": [dict per layer], "gen": the generator, for what follows}."""
    c, H, bf = cfg, cfg.hidden, torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(c.seed)

    def lin(o, i):
        return (torch.randn(o, i, device=dev, generator=g, dtype=torch.float32) * 0.02).to(bf)

    out = {"embed": lin(c.vocab, H), "lm_head": lin(c.vocab, H), "final_norm": torch.ones(H, device=dev, dtype=bf),
           "layers": [], "gen": g}
    for _ in range(c.n_layers):
        L = {}
        L["attn_norm"] = torch.ones(H, device=dev, dtype=bf)
        wq_a = lin(c.q_lora, H)
        L["q_norm"] = torch.ones(c.q_lora, device=dev, dtype=bf)
        L["wq_b"] = lin(HEADS * (c.qk_nope + c.qk_rope), c.q_lora)
        wkv_a = lin(DIM_V + c.qk_rope, H)
        # the two projections of the normalised hidden state share one GEMM: rows [q_a | kv_a]
        L["w_qkv_a"] = torch.cat((wq_a, wkv_a)).contiguous()
        L["wq_a"], L["wkv_a"] = L["w_qkv_a"][:c.q_lora], L["w_qkv_a"][c.q_lora:]
        del wq_a, wkv_a
        L["kv_norm"] = torch.ones(DIM_V, device=dev, dtype=bf)
        L["w_uk"] = (torch.randn(HEADS, c.qk_nope, DIM_V, device=dev, generator=g) * 0.02).to(bf)
        L["w_uv"] = (torch.randn(HEADS, DIM_V, c.v_head, device=dev, generator=g) * 0.02).to(bf)
        L["wo"] = lin(H, HEADS * c.v_head)
        L["ffn_norm"] = torch.ones(H, device=dev, dtype=bf)
        L["router"] = (torch.randn(c.n_experts, H, device=dev, generator=g, dtype=torch.float32) * 0.02).to(bf)
        out["layers"].append(L)
    return out


def expert_shard_stream(cfg: DecoderConfig, dev, rank: int, world: int, gen_shared: torch.Generator):
    """Yields, layer by layer, (routed ExpertWeights of this rank's shard, shared ExpertWeights or None) in row-major
    fp8 with 128x128 block scales: routed experts from a per-rank stream, the shared expert from the replicated one."""
    c = cfg
    ge = torch.Generator(device=dev).manual_seed(c.seed + 1000 + rank)
    el = c.n_experts // world
    for _ in range(c.n_layers):
        w1q, w1s = _quant_experts(el, 2 * c.moe_ffn, c.hidden, dev, ge)
        w2q, w2s = _quant_experts(el, c.hidden, c.moe_ffn, dev, ge)
        shared = None
        if c.shared_expert:
            s1q, s1s = _quant_experts(1, 2 * c.moe_ffn, c.hidden, dev, gen_shared)
            s2q, s2s = _quant_experts(1, c.hidden, c.moe_ffn, dev, gen_shared)
            shared = ExpertWeights(s1q, s1s, s2q, s2s)
        yield ExpertWeights(w1q, w1s, w2q, w2s), shared


def build_weights(cfg: DecoderConfig, dev, rank: int, world: int) -> dict:
    """All weights of one rank in the form the kernels read: dense weights plus, per layer, the expert shard with the
    shared expert stored as one more local expert, tile-major. One bundle can back several ``DecoderRank`` objects
    (different KV placement, same weights)."""
    W = build_dense_weights(cfg, dev)
    for L, (experts, shared) in zip(W["layers"], expert_shard_stream(cfg, dev, rank, world, W["gen"])):
        if shared is not None:
            # the shared expert runs inside the routed pipeline (EpLowLatency fold_shared)
            experts = ExpertWeights.with_shared(experts, shared)
        L["experts"] = experts.to_tiled()   # tile-major: sequential DRAM reads in the fused kernel
        L["shared"] = None
        del experts, shared
    return W


class DecoderRank:
    """One rank's shard of the decoder plus its KV cache, offload manager and EP state."""

    def __init__(self, cfg: DecoderConfig, group: Optional[dist.ProcessGroup] = None, device=None,
                 weights: Optional[dict] = None):
        self.cfg = cfg
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        dev = device or torch.device("cuda", torch.cuda.current_device())
        self.device = dev
        c = cfg
        assert c.n_experts % self.world == 0 and c.ctx % PAGE == 0 and (c.ctx // PAGE) % 2 == 0
        H = c.hidden
        bf = torch.bfloat16
        W = weights if weights is not None else build_weights(c, dev, self.rank, self.world)
        self.weights = W
        self.embed, self.lm_head, self.final_norm, self.layers = W["embed"], W["lm_head"], W["final_norm"], W["layers"]
        # EP state
        nbytes = EpLowLatency.heap_bytes(self.world, c.n_experts, c.top_k, H, c.batch, fold_shared=c.shared_expert)
        self.heap = SymmetricHeap(nbytes, group) if self.world > 1 else SymmetricHeap(nbytes)
        # with the row-gather prefetch running beside it, the persistent MoE kernel leaves a few SMs to the gather
        # (its CTAs take every register of their SM, so the two kernels cannot share one)
        self.gather_ctas = 8
        n_sm = torch.cuda.get_device_properties(dev).multi_processor_count
        moe_ctas = n_sm - self.gather_ctas if (c.offload and c.kv_fetch == "rows") else 0
        self.ep = EpLowLatency(self.heap, c.n_experts, c.top_k, H, c.moe_ffn, c.batch, gemm_ctas=moe_ctas,
                               fold_shared=c.shared_expert)
        # KV cache: pages [0, P/2) resident, [P/2, P) staged from host, page P holds the token being decoded
        B = c.batch
        P = c.ctx // PAGE
        self.pages_per_seq = P + 1
        half = P // 2
        assert c.kv_fetch in ("rows", "pages")
        self.rows_mode = c.offload and c.kv_fetch == "rows"
        self.n_resident = B * (half + 1)
        self.n_staging = B * half            # pages per layer that live in host memory
        # device pages behind the resident ones: the whole offloaded half ("pages"), or topk rows per sequence
        self.land_pages_per_seq = (c.topk_kv + PAGE - 1) // PAGE
        self.n_landing = B * self.land_pages_per_seq if self.rows_mode else self.n_staging
        n_dev_pages = self.n_resident + self.n_landing
        ncol = P + 1 + (self.land_pages_per_seq if self.rows_mode else 0)
        bt = torch.zeros(B, ncol, dtype=torch.int32)
        host_tab = torch.full((B, P + 1), -1, dtype=torch.int32)
        for b in range(B):
            bt[b, :half] = torch.arange(half) + b * (half + 1)
            bt[b, P] = b * (half + 1) + half
            if self.rows_mode:
                # logical pages [half, P) have no device page; selected rows land in the virtual pages behind P
                bt[b, P + 1:] = self.n_resident + b * self.land_pages_per_seq + torch.arange(self.land_pages_per_seq)
            else:
                bt[b, half:P] = self.n_resident + b * half + torch.arange(half)
            host_tab[b, half:P] = b * half + torch.arange(half)
        self.block_table = bt.to(dev)
        self.virt_base = (P + 1) * PAGE
        self.new_page = bt[:, P].to(dev).long()
        self.kv = []
        gk = torch.Generator(device=dev).manual_seed(c.seed + 5000 + self.rank)
        for _ in range(c.n_layers):
            pool = torch.empty(n_dev_pages, PAGE, KV_DIM, device=dev, dtype=bf)
            for s0 in range(0, n_dev_pages, 4096):
                s1 = min(n_dev_pages, s0 + 4096)
                pool[s0:s1] = (torch.randn(s1 - s0, PAGE, KV_DIM, device=dev, generator=gk) * 0.5).to(bf)
            self.kv.append(pool)
        self.kvm = None
        if c.offload:
            page_bytes = PAGE * KV_DIM * 2
            self.kvm = KvOffloadManager(page_bytes, c.n_layers * self.n_staging, channels=c.n_layers)
            self._host_ids = []
            self._host_tab, self._idx_remap = [], []
            if self.rows_mode:
                # the offloaded half is generated chunk by chunk and moved out with cudaMemcpyAsync on the side stream
                chunk = max(1, min(self.n_staging, self.n_landing))
                scratch = torch.empty(chunk, PAGE, KV_DIM, device=dev, dtype=bf)
                for l in range(c.n_layers):
                    for s0 in range(0, self.n_staging, chunk):
                        n = min(chunk, self.n_staging - s0)
                        scratch[:n] = (torch.randn(n, PAGE, KV_DIM, device=dev, generator=gk) * 0.5).to(bf)
                        self.kvm.offload(scratch, list(range(n)),
                                         list(range(l * self.n_staging + s0, l * self.n_staging + s0 + n)))
                        self.kvm.sync()
                    self._host_tab.append((host_tab + torch.where(host_tab >= 0, l * self.n_staging, 0))
                                          .to(torch.int32).to(dev).contiguous())
                    self._idx_remap.append(torch.empty(B, c.topk_kv, dtype=torch.int32, device=dev))
            else:
                self._dev_ids = (ctypes.c_int * self.n_staging)(*range(self.n_resident,
                                                                       self.n_resident + self.n_staging))
                for l in range(c.n_layers):
                    hs = list(range(l * self.n_staging, (l + 1) * self.n_staging))
                    self._host_ids.append((ctypes.c_int * self.n_staging)(*hs))
                    # move the staged half out to pinned host memory (the state every decode step starts from)
                    self.kvm.offload(self.kv[l], list(self._dev_ids), hs)
                self.kvm.sync()
        pos = float(c.ctx)
        inv_freq = 1.0 / (c.rope_theta ** (torch.arange(0, c.qk_rope, 2, device=dev, dtype=torch.float32) / c.qk_rope))
        self.cos = torch.cos(pos * inv_freq)
        self.sin = torch.sin(pos * inv_freq)
        self.sm_scale = 1.0 / math.sqrt(c.qk_nope + c.qk_rope)
        self.attn_status = torch.zeros(4, dtype=torch.int32, device=dev)
        self.new_row = (self.new_page * PAGE).contiguous()      # row (in units of 576 elements) of the new token
        self._o_lat = [torch.empty(B, HEADS, DIM_V, device=dev, dtype=bf) for _ in range(c.n_layers)]
        self._prefetched = False
        # CUDA-graph replay of the step (captured lazily by the first step() after one eager step)
        self.use_graphs = True
        self._graphs = None
        self._steps_run = 0

    # ------------------------------------------------------------------------------------------------------------
    def _rope(self, x: torch.Tensor) -> torch.Tensor:
        x1, x2 = x[..., 0::2].float(), x[..., 1::2].float()
        out = torch.stack((x1 * self.cos - x2 * self.sin, x1 * self.sin + x2 * self.cos), dim=-1)
        return out.flatten(-2).to(x.dtype)

    def prefetch(self, indices: Optional[List[torch.Tensor]] = None, after_compute: bool = True):
        """Queues, on the side stream, the transfers that bring the offloaded KV of every layer back: the rows that
        ``indices`` select (kv_fetch == "rows"; they must be the indices of the next ``step``) or every offloaded
        page ("pages"). ``after_compute=False`` lets the transfers start at once instead of after the work already
        queued on the compute stream; the caller then guarantees that ``indices`` are final (static, or written on
        ``kvm.side_stream()``)."""
        if self.kvm is None:
            return
        for l in range(self.cfg.n_layers):
            if self.rows_mode:
                landing = self.kv[l][self.n_resident:]
                self.kvm.prefetch_rows(l, indices[l], self._host_tab[l], landing, self._idx_remap[l],
                                       self.virt_base, PAGE, status=self.attn_status, after_compute=after_compute,
                                       num_ctas=self.gather_ctas)
            else:
                self.kvm.prefetch(l, self.kv[l], self._dev_ids, self._host_ids[l], self.n_staging)
        self._prefetched = True

    # ---- fused path: torch GEMMs + ops/glue.py kernels --------------------------------------------------------
    def _pre_attn(self, l: int, x: torch.Tensor, a: Optional[torch.Tensor], b: Optional[torch.Tensor]):
        """x + a + b -> (new residual, absorbed query [B, 128, 576]); also writes the new token's KV row."""
        c, L = self.cfg, self.layers[l]
        B = x.shape[0]
        x, h = glue.add_rmsnorm(x, L["attn_norm"], a, b)
        qkv = h @ L["w_qkv_a"].t()
        qa = glue.qkv_post(qkv, c.q_lora, L["q_norm"], L["kv_norm"], self.cos, self.sin, self.kv[l], self.new_row,
                           self.attn_status)
        q = (qa @ L["wq_b"].t()).view(B, HEADS, c.qk_nope + c.qk_rope)
        q_full = torch.empty(B, HEADS, KV_DIM, device=x.device, dtype=x.dtype)
        # absorb W_uk: per head [B, nope] x [nope, 512], written straight into the latent part of q_full
        torch.bmm(q[..., :c.qk_nope].transpose(0, 1), L["w_uk"], out=q_full[..., :DIM_V].transpose(0, 1))
        glue.q_rope(q, c.qk_nope, self.cos, self.sin, q_full)
        return x, q_full

    def _attn(self, l: int, q_full: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
        if self.kvm is not None:
            self.kvm.wait(l)
            if self.rows_mode:
                indices = self._idx_remap[l]
        sparse_mla_decode(q_full, self.kv[l], self.block_table, indices, self.sm_scale, out=self._o_lat[l],
                          status=self.attn_status)
        if self.kvm is not None:
            self.kvm.release(l)
        return self._o_lat[l]

    def _post_attn(self, l: int, x: torch.Tensor, o_lat: torch.Tensor):
        """-> (residual after attention, routed MoE output, shared-expert output or None)."""
        c, L = self.cfg, self.layers[l]
        B = x.shape[0]
        o = torch.empty(B, HEADS, c.v_head, device=x.device, dtype=x.dtype)
        torch.bmm(o_lat.transpose(0, 1), L["w_uv"], out=o.transpose(0, 1))
        x = torch.addmm(x, o.view(B, HEADS * c.v_head), L["wo"].t())
        _, h = glue.add_rmsnorm(x, L["ffn_norm"])
        logits = h @ L["router"].t()
        if c.shared_expert:
            idx, w = glue.router_topk(logits, c.top_k, c.n_experts // self.world, self.rank)
            moe, share, _ = self.ep.moe(h, idx, w, L["experts"], None, prefolded=True)
        else:
            idx, w = glue.router_topk(logits, c.top_k)
            moe, share, _ = self.ep.moe(h, idx, w, L["experts"], L["shared"])
        return x, moe, share

    def _head(self, x, a, b):
        _, h = glue.add_rmsnorm(x, self.final_norm, a, b)
        return torch.argmax(h @ self.lm_head.t(), dim=-1)

    def _capture(self):
        """Records the step as n_layers + 1 CUDA graphs that share one memory pool: [embed .. q of layer 0],
        [after attention l .. q of layer l + 1] for every l, [after the last attention .. sampled tokens]."""
        c = self.cfg
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=self.group)
        self._tok_in = torch.zeros(c.batch, dtype=torch.int64, device=self.device)
        pool = torch.cuda.graph_pool_handle()
        segs, keep = [], []

        def record(fn):
            n0 = _native.LAUNCH_COUNT
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=pool, capture_error_mode="thread_local"):
                res = fn()
            segs.append((g, _native.LAUNCH_COUNT - n0))
            keep.append(res)
            return res

        x, q_full = record(lambda: self._pre_attn(0, self.embed[self._tok_in], None, None))
        q_fulls = [q_full]
        for l in range(c.n_layers - 1):
            def mid(l=l, x=x):
                x2, a, b = self._post_attn(l, x, self._o_lat[l])
                return self._pre_attn(l + 1, x2, a, b)
            x, q_full = record(mid)
            q_fulls.append(q_full)

        def last(x=x):
            x2, a, b = self._post_attn(c.n_layers - 1, x, self._o_lat[c.n_layers - 1])
            return self._head(x2, a, b)
        out = record(last)
        torch.cuda.synchronize()
        self._graphs = dict(segs=segs, q_fulls=q_fulls, out=out, keep=keep)

    def step(self, tokens: torch.Tensor, indices: List[torch.Tensor]) -> torch.Tensor:
        """tokens [B] int64 (device), indices[l] [B, topk_kv] int32 (device) -> next tokens [B] int64 (device).
        With ``use_graphs`` the first call runs eagerly, the second records the graphs, later calls replay them
        (the result then lives in a buffer that the next call overwrites)."""
        if self.kvm is not None and not self._prefetched:
            self.prefetch(indices)
        self._prefetched = False
        self._steps_run += 1
        if self.use_graphs and self._graphs is None and self._steps_run >= 2:
            self._capture()
        if self._graphs is not None:
            G = self._graphs
            self._tok_in.copy_(tokens, non_blocking=True)
            for l in range(self.cfg.n_layers):
                g, n = G["segs"][l]
                g.replay()
                _native.LAUNCH_COUNT += n
                self._attn(l, G["q_fulls"][l], indices[l])
            g, n = G["segs"][-1]
            g.replay()
            _native.LAUNCH_COUNT += n
            return G["out"]
        x, a, b = self.embed[tokens], None, None
        for l in range(self.cfg.n_layers):
            x, q_full = self._pre_attn(l, x, a, b)
            o_lat = self._attn(l, q_full, indices[l])
            x, a, b = self._post_attn(l, x, o_lat)
        return self._head(x, a, b)

    # ---- the same step in plain torch ops (oracle of the fused path) -----------------------------------------
    def _layer_eager(self, l: int, x: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
        c, L = self.cfg, self.layers[l]
        B, H = x.shape
        h = F.rms_norm(x, (H,), L["attn_norm"])
        qa = F.rms_norm(h @ L["wq_a"].t(), (c.q_lora,), L["q_norm"])
        q = (qa @ L["wq_b"].t()).view(B, HEADS, c.qk_nope + c.qk_rope)
        kva = h @ L["wkv_a"].t()
        ckv = F.rms_norm(kva[:, :DIM_V], (DIM_V,), L["kv_norm"])
        krope = self._rope(kva[:, DIM_V:])
        self.kv[l][self.new_page, 0] = torch.cat((ckv, krope), dim=-1)
        q_lat = torch.einsum("bhd,hdc->bhc", q[..., :c.qk_nope], L["w_uk"])
        q_full = torch.cat((q_lat, self._rope(q[..., c.qk_nope:])), dim=-1).contiguous()
        o_lat = self._attn(l, q_full, indices)
        o = torch.einsum("bhc,hcd->bhd", o_lat, L["w_uv"]).reshape(B, HEADS * c.v_head)
        x = x + o @ L["wo"].t()
        h = F.rms_norm(x, (H,), L["ffn_norm"])
        probs = torch.softmax((h @ L["router"].t()).float(), dim=-1)
        w, idx = torch.topk(probs, c.top_k, dim=-1)
        w = (w / w.sum(dim=-1, keepdim=True)).contiguous()
        moe, share, _ = self.ep.moe(h.contiguous(), idx.contiguous(), w, L["experts"], L["shared"])
        x = x + moe
        if share is not None:
            x = x + share
        return x

    def step_eager(self, tokens: torch.Tensor, indices: List[torch.Tensor], return_logits: bool = False):
        if self.kvm is not None and not self._prefetched:
            self.prefetch(indices)
        self._prefetched = False
        x = self.embed[tokens]
        for l in range(self.cfg.n_layers):
            x = self._layer_eager(l, x, indices[l])
        x = F.rms_norm(x, (self.cfg.hidden,), self.final_norm)
        logits = x @ self.lm_head.t()
        return logits if return_logits else torch.argmax(logits, dim=-1)

    def step_logits(self, tokens: torch.Tensor, indices: List[torch.Tensor]) -> torch.Tensor:
        """The fused path without graphs, returning the logits (for comparisons against ``step_eager``)."""
        if self.kvm is not None and not self._prefetched:
            self.prefetch(indices)
        self._prefetched = False
        x, a, b = self.embed[tokens], None, None
        for l in range(self.cfg.n_layers):
            x, q_full = self._pre_attn(l, x, a, b)
            o_lat = self._attn(l, q_full, indices[l])
            x, a, b = self._post_attn(l, x, o_lat)
        _, h = glue.add_rmsnorm(x, self.final_norm, a, b)
        return h @ self.lm_head.t()

    def check(self):
        from ..ops.ep import check_status
        self.ep.check("decoder MoE")
        check_status(self.attn_status, "sparse_mla_decode")

    def close(self):
        if self.kvm is not None:
            self.kvm.close()
        self.heap.close()


def reference_layer_moe(cfg: DecoderConfig, h: torch.Tensor, idx: torch.Tensor, w: torch.Tensor,
                        experts: ExpertWeights) -> torch.Tensor:
    """fp32 oracle of one rank's MoE output when the EP group has a single rank (used by tests)."""
    experts = experts.to_row_major()
    return ref.ref_fused_moe(h, idx, w, experts.w1q, experts.w1s, experts.w2q, experts.w2s)
