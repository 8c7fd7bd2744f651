"""Qwen3 dense on the sm_100a kernels: packed parameters, training forward/backward with
per-layer recomputation, prefill, and single-token decode against a KV cache.

The SAME kernels with the SAME per-row programs serve rollout (decode, batch of sequences) and
training (packed full sequences), which is what makes the selected-token log-probs of the two
bitwise equal.  Every matrix product is ``det_gemm`` (csrc/gemm/det_gemm_sm100.cu); row-parallel
projections use canonical K chunks so the tensor-parallel degree does not change a bit.

Tensor parallelism follows the usual column/row split (rl_engine/backends/cuda/ffn/ffn.py:554-683,
rl_engine/integrations/engines/train/megatron/runtime.py:491-636 in the reference); the partial
sums of row-parallel GEMMs go through ``ParallelContext.tp_all_reduce`` (fixed balanced tree).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from rl_kernel_b200.backends import native as nv
from rl_kernel_b200.models.qwen3.spec import VOCAB_TILE, Qwen3DenseSpec
from rl_kernel_b200.models.qwen3.weights import (Qwen3DenseWeights, pack_gate_up, pack_qkv, pad_vocab,
                                                 unpack_gate_up, unpack_qkv)

BF16 = torch.bfloat16


# ------------------------------------------------------------------------------ parallel context
class ParallelContext:
    """Rank geometry plus the collectives the engine needs.  The default is a single GPU."""

    def __init__(self, tp_rank: int = 0, tp_size: int = 1, cp_rank: int = 0, cp_size: int = 1,
                 collective=None, cp_collective=None):
        self.tp_rank, self.tp_size = tp_rank, tp_size
        self.cp_rank, self.cp_size = cp_rank, cp_size
        self.collective = collective        # fixed-order TP collective (all_reduce_, all_gather)
        self.cp_collective = cp_collective
        # data parallel replicas (each trains its own sequences; gradients are summed over them)
        self.dp_rank, self.dp_size, self.dp_collective = 0, 1, None
        self.tp_group = self.cp_group = self.dp_group = None

    def tp_all_reduce_(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp_size > 1:
            self.collective.all_reduce_(x)
        return x

    def tp_all_gather(self, x: torch.Tensor) -> torch.Tensor:
        """[..] -> [tp, ..] in rank order."""
        if self.tp_size == 1:
            return x.unsqueeze(0)
        return self.collective.all_gather(x)


# ------------------------------------------------------------------------------ parameters
@dataclass
class _Slot:
    name: str
    shape: tuple[int, ...]
    offset: int = 0

    @property
    def numel(self) -> int:
        return math.prod(self.shape)


class PackedParams:
    """All parameters of one rank in ONE flat bf16 buffer (plus a twin for gradients), so the
    optimizer, gradient clipping, weight sync and gradient all-reduce are single launches."""

    def __init__(self, spec: Qwen3DenseSpec, tp_rank: int, tp_size: int, device: torch.device,
                 with_grad: bool = False, *, layers: tuple[int, int] | None = None,
                 has_embed: bool = True, has_head: bool = True, storage: torch.Tensor | None = None):
        """``layers`` = (first, end) and ``has_embed`` / ``has_head`` select what a pipeline stage owns
        (default: the whole model).  ``storage``: an existing flat bf16 tensor of at least ``numel``
        elements to place the parameters in (its contents are kept)."""
        if spec.canonical_tp % tp_size:
            raise ValueError(f"tp_size {tp_size} must divide canonical_tp {spec.canonical_tp}")
        self.spec, self.tp_rank, self.tp_size, self.device = spec, tp_rank, tp_size, device
        self.layer_range = layers if layers is not None else (0, spec.num_hidden_layers)
        self.has_embed, self.has_head = has_embed, has_head
        h, d = spec.hidden_size, spec.head_dim
        self.qkv_local = spec.qkv_dim // tp_size
        self.q_local = spec.q_dim // tp_size
        self.kv_local = spec.kv_dim // tp_size
        self.i_local = spec.intermediate_size // tp_size
        self.v_local = spec.padded_vocab_size // tp_size
        self.vocab_start = tp_rank * self.v_local
        self.v_real_local = max(0, min(self.v_local, spec.vocab_size - self.vocab_start))
        slots: list[_Slot] = [_Slot("embed", (self.v_local, h))] if has_embed else []
        for l in range(*self.layer_range):
            slots += [_Slot(f"l{l}.ln1", (h,)), _Slot(f"l{l}.wqkv", (self.qkv_local, h)),
                      _Slot(f"l{l}.qn", (d,)), _Slot(f"l{l}.kn", (d,)),
                      _Slot(f"l{l}.wo", (h, self.q_local)), _Slot(f"l{l}.ln2", (h,))]
            slots += self._mlp_slots(l)
        if has_head:
            slots += [_Slot("norm", (h,)), _Slot("lm_head", (self.v_local, h))]
        slots += self._trailing_slots()
        off = 0
        for s in slots:
            s.offset = off
            off += (s.numel + 7) // 8 * 8
        self.slots = {s.name: s for s in slots}
        self.numel = off
        if storage is not None:
            if storage.dtype != BF16 or storage.numel() < off or not storage.is_contiguous():
                raise ValueError("storage must be a contiguous bf16 tensor of at least numel elements")
            self.flat = storage[:off]
        else:
            self.flat = torch.zeros(off, dtype=BF16, device=device)
        self.grad = torch.zeros(off, dtype=BF16, device=device) if with_grad else None
        self.w = {s.name: self.flat[s.offset:s.offset + s.numel].view(s.shape) for s in slots}
        self.g = ({s.name: self.grad[s.offset:s.offset + s.numel].view(s.shape) for s in slots}
                  if with_grad else {})

    def _mlp_slots(self, l: int) -> list[_Slot]:
        h = self.spec.hidden_size
        return [_Slot(f"l{l}.wgu", (2 * self.i_local, h)), _Slot(f"l{l}.wd", (h, self.i_local))]

    def _trailing_slots(self) -> list[_Slot]:
        """Slots placed after everything else (subclasses: parameters that are not replicated over
        the data-parallel group, so that the replicated ones form one contiguous prefix)."""
        return []

    # replicated (not TP-sharded) parameters: their gradients are identical on every TP rank
    def is_replicated(self, name: str) -> bool:
        return name.endswith((".ln1", ".ln2", ".qn", ".kn")) or name == "norm"

    def load(self, weights: Qwen3DenseWeights) -> "PackedParams":
        spec, r, tp = self.spec, self.tp_rank, self.tp_size
        dev = self.device

        def put(name: str, t: torch.Tensor) -> None:
            self.w[name].copy_(t.to(device=dev, dtype=BF16))

        def rows(t: torch.Tensor) -> torch.Tensor:
            n = t.shape[0] // tp
            return t[r * n:(r + 1) * n]

        def cols(t: torch.Tensor) -> torch.Tensor:
            n = t.shape[1] // tp
            return t[:, r * n:(r + 1) * n]

        if self.has_embed:
            put("embed", rows(pad_vocab(spec, weights["embed_tokens.weight"])))
        if self.has_head:
            put("lm_head", rows(pad_vocab(spec, weights["lm_head.weight"])))
            put("norm", weights["norm.weight"])
        for l in range(*self.layer_range):
            p = f"layers.{l}"
            put(f"l{l}.ln1", weights[f"{p}.input_layernorm.weight"])
            put(f"l{l}.ln2", weights[f"{p}.post_attention_layernorm.weight"])
            put(f"l{l}.qn", weights[f"{p}.self_attn.q_norm.weight"])
            put(f"l{l}.kn", weights[f"{p}.self_attn.k_norm.weight"])
            put(f"l{l}.wqkv", rows(pack_qkv(spec, weights[f"{p}.self_attn.q_proj.weight"],
                                            weights[f"{p}.self_attn.k_proj.weight"],
                                            weights[f"{p}.self_attn.v_proj.weight"])))
            put(f"l{l}.wo", cols(weights[f"{p}.self_attn.o_proj.weight"]))
            put(f"l{l}.wgu", rows(pack_gate_up(spec, weights[f"{p}.mlp.gate_proj.weight"],
                                               weights[f"{p}.mlp.up_proj.weight"])))
            put(f"l{l}.wd", cols(weights[f"{p}.mlp.down_proj.weight"]))
        return self

    def init_synthetic_(self, seed: int = 0, std: float = 0.02) -> "PackedParams":
        """Random-init directly on the device (used for the full-size benchmark where building
        the HF-layout dictionary on the host first would take minutes)."""
        gen = torch.Generator(device=self.device).manual_seed(seed * 1000 + self.tp_rank)
        for name, s in self.slots.items():
            if len(s.shape) == 1:
                self.w[name].fill_(1.0)
            else:
                w = self.w[name]
                step = max(1, (1 << 26) // max(1, w.shape[1]))
                for r0 in range(0, w.shape[0], step):
                    blk = w[r0:r0 + step]
                    blk.copy_(torch.randn(blk.shape, generator=gen, device=self.device,
                                          dtype=torch.float32).mul_(std))
        for name in ("embed", "lm_head"):
            if name in self.w and self.v_real_local < self.v_local:
                self.w[name][self.v_real_local:].zero_()
        return self

    def export_local(self, table: dict[str, torch.Tensor] | None = None) -> dict[str, torch.Tensor]:
        """This rank's shard back in HF key names (TP=1: the full HF state).  ``table``: the packed tensors to read
        (default the weights ``self.w``; ``self.g`` gives the gradients under the same names)."""
        spec = self.spec
        W = self.w if table is None else table
        if self.tp_size != 1:
            raise NotImplementedError("export_local assembles full tensors only for tp_size == 1")
        out = {"embed_tokens.weight": W["embed"][:spec.vocab_size],
               "lm_head.weight": W["lm_head"][:spec.vocab_size], "norm.weight": W["norm"]}
        for l in range(spec.num_hidden_layers):
            p = f"layers.{l}"
            q, k, v = unpack_qkv(spec, W[f"l{l}.wqkv"])
            gte, up = unpack_gate_up(spec, W[f"l{l}.wgu"])
            out.update({f"{p}.input_layernorm.weight": W[f"l{l}.ln1"],
                        f"{p}.post_attention_layernorm.weight": W[f"l{l}.ln2"],
                        f"{p}.self_attn.q_norm.weight": W[f"l{l}.qn"],
                        f"{p}.self_attn.k_norm.weight": W[f"l{l}.kn"],
                        f"{p}.self_attn.q_proj.weight": q, f"{p}.self_attn.k_proj.weight": k,
                        f"{p}.self_attn.v_proj.weight": v,
                        f"{p}.self_attn.o_proj.weight": W[f"l{l}.wo"],
                        f"{p}.mlp.gate_proj.weight": gte, f"{p}.mlp.up_proj.weight": up,
                        f"{p}.mlp.down_proj.weight": W[f"l{l}.wd"]})
        return out

    def export_local_grads(self) -> dict[str, torch.Tensor]:
        """Gradients in HF key names (needs ``with_grad=True``; TP=1)."""
        if self.grad is None:
            raise RuntimeError("these parameters were built without a gradient buffer")
        return self.export_local(self.g)


# ------------------------------------------------------------------------------ attention tiles
def rope_tables(spec: Qwen3DenseSpec, max_pos: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    d = spec.head_dim
    inv_freq = 1.0 / (spec.rope_theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv_freq[None]
    return (ang.cos().float().to(device).contiguous(), ang.sin().float().to(device).contiguous())


def train_tiles(nseq: int, S: int, hq: int, hkv: int, d: int, device, *, q_pos0: int = 0
                ) -> tuple[torch.Tensor, torch.Tensor]:
    """Forward/dQ tiles and dK/dV tiles for ``nseq`` packed sequences of length ``S``."""
    g = hq // hkv
    nqt = (S + 127) // 128
    b = torch.arange(nseq).view(-1, 1, 1)
    qt = torch.arange(nqt - 1, -1, -1).view(1, -1, 1)  # longest tiles first
    h = torch.arange(hq).view(1, 1, -1)
    z = torch.zeros(nseq, nqt, hq, dtype=torch.long)
    row0 = b * S + qt * 128 + z
    fw = torch.stack([row0, h * d + z, torch.clamp(S - qt * 128, max=128) + z, b * S + z,
                      (h // g) * d + z, qt * 128 + q_pos0 + z, z + 1, z + S + q_pos0,
                      row0 * hq + h, z + hq, z, z], dim=-1).reshape(-1, 12)
    hk = torch.arange(hkv).view(1, 1, -1)
    kb = torch.arange(nqt).view(1, -1, 1)
    zk = torch.zeros(nseq, nqt, hkv, dtype=torch.long)
    kv = torch.stack([b * S + kb * 128 + zk, hk * d + zk, kb * 128 + zk,
                      torch.clamp(S - kb * 128, max=128) + zk, b * S + zk, zk + q_pos0, zk + S,
                      hk * g * d + zk, zk + g, (b * S) * hq + hk * g + zk, zk + hq, zk + 1],
                     dim=-1).reshape(-1, 12)
    return fw.to(torch.int32).to(device).contiguous(), kv.to(torch.int32).to(device).contiguous()


# ------------------------------------------------------------------------------ workspace
class Workspace:
    """Named, shape-keyed scratch tensors that live for the lifetime of the engine.

    With an ``arena`` (one big uint8 tensor) the buffers whose names start with one of
    ``arena_prefixes`` are carved out of it by a bump allocator instead of being allocated one by
    one.  The GRPO trainer hands the same arena to the KV cache: rollout and training never run at
    the same time, so the training activations reuse the cache's memory (the cache is re-zeroed
    before every rollout)."""

    def __init__(self, device, arena: torch.Tensor | None = None,
                 arena_prefixes: tuple[str, ...] = ("f.", "r.", "b.", "lm.", "ckpt", "pos", "act")):
        self.device = device
        self._bufs: dict[tuple, torch.Tensor] = {}
        self.arena, self.arena_prefixes, self._off = arena, arena_prefixes, 0

    def get(self, name: str, shape: tuple[int, ...], dtype=BF16, zero: bool = False) -> torch.Tensor:
        key = (name, tuple(shape), dtype)
        t = self._bufs.get(key)
        if t is None:
            nbytes = math.prod(shape) * torch.empty((), dtype=dtype).element_size()
            if (self.arena is not None and name.startswith(self.arena_prefixes)
                    and self._off + nbytes <= self.arena.numel()):
                t = self.arena[self._off:self._off + nbytes].view(dtype).view(shape)
                self._off = (self._off + nbytes + 255) // 256 * 256
                if zero:
                    t.zero_()
            else:
                t = (torch.zeros if zero else torch.empty)(shape, dtype=dtype, device=self.device)
            self._bufs[key] = t
        return t

    def release(self, prefix: str = "") -> None:
        for k in [k for k in self._bufs if k[0].startswith(prefix)]:
            del self._bufs[k]

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._bufs.values())


@dataclass
class KVCache:
    k: list[torch.Tensor]   # per layer [nseq * max_len, kv_local]
    v: list[torch.Tensor]
    nseq: int
    max_len: int
    flat: torch.Tensor | None = None   # the single buffer behind k and v (for one-shot zeroing)


@dataclass
class _Leaves:
    """Per-chunk partial results of a few-row row-parallel GEMM whose tree the next norm evaluates."""
    buf: torch.Tensor
    stride: int
    nchunks: int


@dataclass
class SharedPrefixKV:
    """KV pool in which the sequences of a GRPO group share their prompt's pages: per layer
    [num_prompts * P + nseq * R_pad, kv_local] rows = prompt region then one response region per
    sequence, addressed through a page table (page = 128 rows)."""
    kv: KVCache                 # the whole pool (nseq = 1, max_len = rows)
    prompt_kv: KVCache          # view of the prompt region, [num_prompts, P] (prefill writes here)
    page_table: torch.Tensor    # int32 [nseq, blocks_per_seq]
    slot_base: torch.Tensor     # int32 [nseq]: pool row of a sequence's first response token
    prompt_len: int
    blocks_per_seq: int
    seq_of_tile: torch.Tensor | None = None
    # prompt blocks attended once per (prompt, KV head) for the whole group; the per-sequence
    # tiles resume from the saved row state (decode_tiles_shared_prefix fills these)
    prefix_tiles: torch.Tensor | None = None
    prefix_ext: torch.Tensor | None = None
    seq_ext: torch.Tensor | None = None
    row_state: torch.Tensor | None = None
    group: int = 0


@dataclass
class TrainState:
    nseq: int
    S: int
    ckpt: torch.Tensor                      # [L, T, H] residual-stream input of every layer
    last_x: torch.Tensor | None = None      # output of the last MLP (pre residual add)
    last_res: torch.Tensor | None = None
    final_s: torch.Tensor | None = None
    extra: dict = field(default_factory=dict)


class Qwen3Engine:
    """Forward / backward / decode of one model replica shard on one GPU."""

    def __init__(self, spec: Qwen3DenseSpec, params: PackedParams, ctx: ParallelContext | None = None,
                 max_positions: int = 4096):
        self.spec, self.p = spec, params
        self.ctx = ctx or ParallelContext()
        self.dev = params.device
        tp = self.ctx.tp_size
        self.hq = spec.num_attention_heads // tp
        self.hkv = spec.num_key_value_heads // tp
        self.d = spec.head_dim
        if self.d != 128:
            raise ValueError("the sm_100a attention kernels are specialised for head_dim 128")
        self.l0, self.l1 = params.layer_range        # decoder layers of this pipeline stage
        self.first_stage, self.last_stage = params.has_embed, params.has_head
        self.nchunks = spec.canonical_tp // tp      # canonical K chunks held by this rank
        self.blk = spec.intermediate_size // spec.canonical_tp
        self.scale = 1.0 / math.sqrt(self.d)
        self.cos, self.sin = rope_tables(spec, max_positions, self.dev)
        self.ws = Workspace(self.dev)
        # Row-parallel projections with many rows: the GEMM writes its partial into the symmetric
        # frame and the two-shot all-reduce kernel follows (False), or one fused kernel pulls the
        # peers' tiles in its epilogue (True).  Measured on two GPUs at 12288 x 4096 outputs the
        # fused kernel loses (0.78 against 0.49 ms at K = 2048 per rank): its one-shot pulls move
        # (W - 1) x the tile over NVLink inside the epilogue, 25 us per tile, which the mainloop
        # cannot hide.
        self.fuse_gemm_allreduce = False
        # Layout-invariant parameter gradients: q_norm / k_norm gains as a tree over KV groups, the LM
        # head's input gradient over canonical vocabulary chunks.  With them every gradient of a
        # tensor-parallel run equals the single-GPU gradient bit for bit.
        self.canonical_grads = True
        # Under context parallelism the same holds for every parameter: the per-token operands of a gradient are
        # brought into logical token order and each CP rank computes a row slice of the gradient over ALL tokens
        # (distributed/algorithms/canonical_cp.py); the LM head runs vocabulary-parallel over the CP group.  The
        # rows a rank does not own stay zero, so the sum over the CP group assembles the exact single-GPU gradient.
        self.cp_canonical_grads = True
        self.cp = None                               # CPAttention once enable_context_parallel ran
        self._decode_page_table = None               # set while a paged decode step runs
        self._decode_shared = None                   # SharedPrefixKV whose prompt blocks are attended per group
        self.group_prefix_attention = True           # False: every sequence walks its prompt blocks itself
        self._tiles: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}
        for K in (params.q_local, params.i_local):
            if self.nchunks > 1 and (K // self.nchunks) % 64:
                raise ValueError(f"canonical K chunk {K // self.nchunks} must be a multiple of 64")

    def enable_context_parallel(self, max_local_tokens: int, layout: str = "zigzag") -> None:
        """Training over ``ctx.cp_size`` ranks that each hold 1/cp of every sequence: K/V (and Q, dO,
        lse, delta for backward) live in peer-mapped buffers and the attention kernels fetch remote
        blocks themselves (distributed/cp_attention.py)."""
        from rl_kernel_b200.distributed.cp_attention import CPAttention

        if self.ctx.cp_size > 1 and self.cp is None:
            self.cp = CPAttention(self.ctx.cp_collective, self.dev, num_q_heads=self.hq, num_kv_heads=self.hkv,
                                  max_local_tokens=max_local_tokens, layout=layout)

    # -------------------------------------------------------------------------- canonical CP gradients
    @property
    def _cp_canon(self) -> bool:
        return self.cp is not None and self.canonical_grads and self.cp_canonical_grads

    def _cp_order(self, nseq: int, S: int) -> torch.Tensor:
        """Row of the rank-major gathered token tensor that holds logical token (sequence, position)."""
        key = ("cp_order", nseq, S)
        if key not in self._tiles:
            from rl_kernel_b200.distributed.algorithms.canonical_cp import uniform_gather_indices

            self._tiles[key] = (uniform_gather_indices(nseq, S, self.ctx.cp_size, self.cp.layout).to(self.dev), None)
        return self._tiles[key][0]

    def _cp_gather(self, t: torch.Tensor, name: str, cp_geom) -> torch.Tensor:
        """t [T_local, C] of this rank's tokens -> [nseq * S, C] of all tokens in logical order."""
        nseq, S = cp_geom
        g = self.ctx.cp_collective.all_gather(t.contiguous())            # [cp, T_local, C], bits unchanged
        out = self.ws.get(name, (nseq * S, t.shape[1]), t.dtype)
        torch.index_select(g.view(-1, t.shape[1]), 0, self._cp_order(nseq, S), out=out)
        return out

    def _cp_rows(self, n_rows: int) -> tuple[int, int]:
        """The rows of an [n_rows, *] gradient this CP rank computes (equal slices on 128-row boundaries)."""
        cp, r = self.ctx.cp_size, self.ctx.cp_rank
        per = -(-(-(-n_rows // cp)) // 128) * 128
        lo = min(n_rows, r * per)
        return lo, min(n_rows, lo + per)

    def _dw(self, dy, x, grad, *, M: int, N: int, T: int, cp_geom=None) -> None:
        """grad [M, N] += dy [T, M]^T @ x [T, N], tokens reduced in logical order."""
        if cp_geom is None or not self._cp_canon:
            self._gemm(dy, x, grad, a_mn=True, b_mn=True, accumulate=True, M=M, N=N, K=T)
            return
        dyg = self._cp_gather(dy, "cpg.dy", cp_geom)
        xg = self._cp_gather(x, "cpg.x", cp_geom)
        lo, hi = self._cp_rows(M)
        if hi > lo:
            self._gemm(dyg[:, lo:hi], xg, grad[lo:hi], a_mn=True, b_mn=True, accumulate=True, M=hi - lo, N=N,
                       K=dyg.shape[0])

    def _gain_bwd(self, x, w, dy, dx, scr, eps, grad, *, dres=None, owner: int = 0, cp_geom=None) -> None:
        """RMSNorm backward; the gain gradient is accumulated into ``grad`` (under canonical CP by one owner rank,
        from the gathered rows in logical order; the owner rotates over the norms to spread the extra pass)."""
        if cp_geom is None or not self._cp_canon:
            nv.rmsnorm_bwd(x, w, dy, dx, scr, eps, dres=dres, dw_bf16=grad, accumulate_dw=True)
            return
        H = x.shape[1]
        nv.rmsnorm_bwd(x, w, dy, dx, scr, eps, dres=dres, dw_bf16=self.ws.get("cpg.dw_dummy", (H,)), accumulate_dw=False)
        xg = self._cp_gather(x, "cpg.nx", cp_geom)
        dyg = self._cp_gather(dy, "cpg.ndy", cp_geom)
        if owner % self.ctx.cp_size == self.ctx.cp_rank:
            Tg = xg.shape[0]
            scr_g = self.ws.get("cpg.scr", (nv.rmsnorm_bwd_scratch_elems(Tg, H),), torch.float32)
            nv.rmsnorm_bwd(xg, w, dyg, self.ws.get("cpg.ndx", (Tg, H)), scr_g, eps, dw_bf16=grad, accumulate_dw=True)

    # -------------------------------------------------------------------------- helpers
    def _gemm(self, a, b, out, *, a_mn=False, b_mn=False, nchunks=1, accumulate=False, M=None, N=None, K=None):
        if M is None:
            M = a.shape[1] if a_mn else a.shape[0]
            K = a.shape[0] if a_mn else a.shape[1]
            N = b.shape[1] if b_mn else b.shape[0]
        if nchunks > 1 and M <= 512 and not (a_mn or b_mn or accumulate):
            # few rows (decode): one set of CTAs per canonical chunk, then the tree kernel
            scratch = self.ws.get("d.split", (nchunks * M * out.stride(0),))
            return nv.det_gemm_split(a, b, out, scratch, nchunks=nchunks, tile_n=64)
        return nv.det_gemm(a, b, out, M=M, N=N, K=K, a_mn=a_mn, b_mn=b_mn, nchunks=nchunks,
                           accumulate=accumulate)

    fold_tree_into_norm = True     # decode: the chunk tree of o_proj / down is evaluated by the next norm
    fuse_decode_swiglu = True      # decode: the gate/up GEMM writes the SwiGLU output directly

    def _row_parallel_leaves(self, a, w, name: str, nchunks: int) -> _Leaves:
        M, N = a.shape[0], w.shape[0]
        buf = self.ws.get(name, (nchunks * M * N,))
        stride = nv.det_gemm_split_leaves(a, w, buf, nchunks=nchunks, tile_n=64)
        return _Leaves(buf, stride, nchunks)

    def _norm_after(self, x, weight, y, res, res_out):
        """rmsnorm(x + res) where ``x`` may still be in per-chunk form."""
        eps = self.spec.rms_norm_eps
        if isinstance(x, _Leaves):
            nv.rmsnorm_fwd_leaves(x.buf, x.stride, x.nchunks, res, weight, y, res_out, eps)
        else:
            nv.rmsnorm_fwd(x, weight, y, eps, res=res, res_out=res_out)

    def _row_parallel(self, a, w, out, nchunks: int):
        """Row-parallel projection: local GEMM with canonical chunks, then the fixed-tree sum over TP.
        Many rows: one fused GEMM+all-reduce kernel.  Few rows (decode): the split GEMM writes into
        the symmetric frame and the all-reduce kernel skips its copy-in."""
        coll = self.ctx.collective
        if self.ctx.tp_size == 1:
            return self._gemm(a, w, out, nchunks=nchunks)
        M = a.shape[0]
        if M > 512 and hasattr(coll, "gemm_all_reduce") and self.fuse_gemm_allreduce:
            return coll.gemm_all_reduce(a, w, out, nchunks)
        if hasattr(coll, "staging_view"):
            staged = coll.staging_view(tuple(out.shape), out.dtype)
            self._gemm(a, w, staged, nchunks=nchunks)
            return coll.all_reduce_staged(staged, out)
        self._gemm(a, w, out, nchunks=nchunks)
        coll.all_reduce_(out)
        return out

    def _qk_grad_view(self) -> torch.Tensor:
        """[layers, 256] view of the q_norm | k_norm gain gradients inside the flat gradient buffer
        (the two slots are adjacent and every layer has the same slots)."""
        if getattr(self, "_qk_view", None) is None:
            sl = self.p.slots
            first, L = sl[f"l{self.l0}.qn"], self.l1 - self.l0
            assert sl[f"l{self.l0}.kn"].offset == first.offset + 128
            stride = sl[f"l{self.l0 + 1}.qn"].offset - first.offset if L > 1 else 256
            self._qk_view = torch.as_strided(self.p.grad, (L, 256), (stride, 1), first.offset)
        return self._qk_view

    def _qk_stage(self) -> torch.Tensor:
        return self.ws.get("g.qk_stage", (self.l1 - self.l0, 256))

    def _tiles_for(self, nseq: int, S: int):
        key = (nseq, S)
        if key not in self._tiles:
            self._tiles[key] = train_tiles(nseq, S, self.hq, self.hkv, self.d, self.dev)
        return self._tiles[key]

    # -------------------------------------------------------------------------- layer forward
    def _layer_fwd(self, *args, **kwargs):
        """One decoder layer (see ``_layer_fwd_body``).  Every GEMM of the layer multiplies by a
        weight and follows a norm / rope / attention / activation kernel, none of which writes
        weights, so the GEMMs may stream their weights ahead of the dependency wait."""
        with nv.static_weights():
            return self._layer_fwd_body(*args, **kwargs)

    def _layer_fwd_body(self, l: int, x, res, T: int, pos, *, tiles, kbuf, vbuf, kv_slot=None,
                        q_view=None, lse=None, s_in_out=None, keep: dict | None = None, tag: str = "f",
                        cp_geom: tuple[int, int] | None = None, store_tag: str | None = None):
        """One decoder layer.  ``x`` + ``res`` -> (mlp_out, s_mid).  When ``res`` is None, ``x`` is
        already the residual stream.  ``keep`` receives the intermediates backward needs.
        ``store_tag``: the tensors backward cannot cheaply rebuild (qkv, q, attention output, s_mid,
        gate/up) go to buffers of their own under this tag instead of the shared scratch, so they
        survive until this layer's backward."""
        w, ws, H = self.p.w, self.ws, self.spec.hidden_size
        eps = self.spec.rms_norm_eps
        stag = store_tag or tag
        h = ws.get(f"{tag}.h", (T, H))
        if res is None:
            s_in = x
            nv.rmsnorm_fwd(s_in, w[f"l{l}.ln1"], h, eps)
        else:
            s_in = s_in_out if s_in_out is not None else ws.get(f"{tag}.s_in", (T, H))
            self._norm_after(x, w[f"l{l}.ln1"], h, res, s_in)
        qkv = ws.get(f"{stag}.qkv", (T, self.p.qkv_local))
        self._gemm(h, w[f"l{l}.wqkv"], qkv)
        if cp_geom is not None and keep is not None:
            q = self.cp.bufs.local("q")[:T]          # the dK/dV kernels of the peers read it
        else:
            q = ws.get(f"{stag}.q", (T, self.p.q_local))
        nv.qk_norm_rope_fwd(qkv, w[f"l{l}.qn"], w[f"l{l}.kn"], self.cos, self.sin, pos, q, kbuf, vbuf,
                            Hq=self.hq, Hkv=self.hkv, eps=eps, kv_slot=kv_slot)
        attn = ws.get(f"{stag}.attn", (T, self.p.q_local))
        qv = q if q_view is None else q.view(*q_view)
        ov = attn if q_view is None else attn.view(*q_view)
        if cp_geom is not None:
            self.cp.forward_inplace(q, attn, lse, *cp_geom)
        else:
            self._attention(qv, kbuf, vbuf, ov, lse, tiles, decode=q_view is not None)
        fold = (self.fold_tree_into_norm and tag == "d" and self.ctx.tp_size == 1 and self.nchunks > 1 and T <= 512)
        if fold:
            o = self._row_parallel_leaves(attn, w[f"l{l}.wo"], "d.leaf_o", self.nchunks)
        else:
            o = ws.get(f"{tag}.o", (T, H))
            self._row_parallel(attn, w[f"l{l}.wo"], o, self.nchunks)
        s_mid = ws.get(f"{stag}.s_mid", (T, H))
        h2 = ws.get(f"{tag}.h2", (T, H))
        self._norm_after(o, w[f"l{l}.ln2"], h2, s_in, s_mid)
        if keep is not None:
            keep.update(s_in=s_in, h=h, qkv=qkv, q=q, attn=attn, s_mid=s_mid, h2=h2)
        down = self._mlp_fwd(l, h2, T, tag, keep, store_tag)
        return down, s_mid

    supports_stored_activations = True

    def _mlp_fwd(self, l: int, h2: torch.Tensor, T: int, tag: str, keep: dict | None,
                 store_tag: str | None = None) -> torch.Tensor:
        """Feed-forward block on the normalised stream ``h2`` [T, H] -> [T, H] (before the residual)."""
        w, ws, H = self.p.w, self.ws, self.spec.hidden_size
        act = ws.get(f"{tag}.act", (T, self.p.i_local))
        if tag == "d" and keep is None and T <= 128 and self.blk % 96 == 0 and self.fuse_decode_swiglu:
            # decode: SwiGLU in the epilogue of the gate/up GEMM (nobody needs the gate/up tensor)
            gu = None
            nv.det_gemm_swiglu(h2, w[f"l{l}.wgu"], act, self.blk)
        else:
            gu = ws.get(f"{store_tag or tag}.gu", (T, 2 * self.p.i_local))
            self._gemm(h2, w[f"l{l}.wgu"], gu)
            nv.swiglu_fwd(gu, act, self.p.i_local, self.blk)
        if self.fold_tree_into_norm and tag == "d" and self.ctx.tp_size == 1 and self.nchunks > 1 and T <= 512:
            return self._row_parallel_leaves(act, w[f"l{l}.wd"], "d.leaf_down", self.nchunks)
        down = ws.get(f"{tag}.down", (T, H))
        self._row_parallel(act, w[f"l{l}.wd"], down, self.nchunks)
        if keep is not None:
            keep.update(gu=gu, act=act)
        return down

    def _rebuild_mlp_activation(self, keep: dict, T: int) -> None:
        """Stored-activation backward: SwiGLU output from the kept gate/up tensor."""
        keep["act"] = self.ws.get("r.act", (T, self.p.i_local))
        nv.swiglu_fwd(keep["gu"], keep["act"], self.p.i_local, self.blk)

    def _mlp_bwd(self, l: int, ds: torch.Tensor, keep: dict, T: int, cp_geom=None) -> torch.Tensor:
        """Backward of ``_mlp_fwd``: ``ds`` = d(loss)/d(output) -> d(loss)/d(h2), summed over TP;
        weight gradients are accumulated."""
        w, g, ws, H = self.p.w, self.p.g, self.ws, self.spec.hidden_size
        dact = ws.get("b.dact", (T, self.p.i_local))
        self._gemm(ds, w[f"l{l}.wd"], dact, b_mn=True, M=T, N=self.p.i_local, K=H)
        self._dw(ds, keep["act"], g[f"l{l}.wd"], M=H, N=self.p.i_local, T=T, cp_geom=cp_geom)
        dgu = ws.get("b.dgu", (T, 2 * self.p.i_local))
        nv.swiglu_bwd(keep["gu"], dact, dgu, self.p.i_local, self.blk)
        dh2 = ws.get("b.dh", (T, H))
        self._gemm(dgu, w[f"l{l}.wgu"], dh2, b_mn=True, nchunks=self.nchunks, M=T, N=H,
                   K=2 * self.p.i_local)
        self.ctx.tp_all_reduce_(dh2)
        self._dw(dgu, keep["h2"], g[f"l{l}.wgu"], M=2 * self.p.i_local, N=H, T=T, cp_geom=cp_geom)
        return dh2

    def _attention(self, q2d, k2d, v2d, o2d, lse, tiles, decode: bool = False):
        sp = self._decode_shared if decode else None
        if sp is not None and sp.prefix_tiles is not None and self.group_prefix_attention:
            # The group's rows walk the shared prompt blocks together (one K/V fetch and one MMA
            # chain per block for all samples), save their running softmax state, and every
            # sequence resumes from it on its own response blocks: per row the same block
            # updates in the same order as an uninterrupted run.
            g = self.hq // self.hkv
            nv.attn_fwd(q2d, [k2d], [v2d], o2d, None, sp.prefix_tiles, self.scale, decode=True,
                        page_table=sp.page_table, resume=(sp.prefix_ext, sp.row_state, g, self.hq, sp.group))
            nv.attn_fwd(q2d, [k2d], [v2d], o2d, lse, tiles, self.scale, decode=True,
                        page_table=sp.page_table, resume=(sp.seq_ext, sp.row_state, g, self.hq, 0))
            return
        nv.attn_fwd(q2d, [k2d], [v2d], o2d, lse, tiles, self.scale,
                    decode=decode and self.hq // self.hkv <= 8,
                    page_table=self._decode_page_table if decode else None)

    # -------------------------------------------------------------------------- full forward
    def forward_hidden(self, tokens: torch.Tensor, *, save: TrainState | None = None,
                       kv: KVCache | None = None, tag: str = "f", cp_seq_len: int | None = None,
                       stage_in: tuple[torch.Tensor, torch.Tensor] | None = None):
        """tokens [nseq, S] -> final-norm hidden [nseq*S, H].  With ``kv`` the K/V of every layer are
        written into the cache (prefill); with ``save`` layer inputs are checkpointed for backward.
        ``cp_seq_len``: context parallel -- ``tokens`` holds this rank's S = cp_seq_len / cp positions
        of every sequence (``cp.local_positions`` order).
        Pipeline stages: a stage without the embedding takes ``stage_in`` = (block output, residual)
        of the previous stage's last layer; a stage without the head returns that pair for its own
        last layer instead of the final-norm hidden (the pair, not its sum, crosses the boundary so
        that the next layer's fused add + norm sees exactly the single-GPU operands)."""
        nseq, S = tokens.shape
        T, H = nseq * S, self.spec.hidden_size
        if (kv is not None or cp_seq_len is not None) and not (self.first_stage and self.last_stage):
            raise NotImplementedError("KV-cache and context-parallel paths run on a whole-model engine")
        ws = self.ws
        pos = ws.get("pos" if tag == "f" else f"{tag}.pos", (T,), torch.int32)
        cp_geom = None
        if cp_seq_len is not None:
            if self.cp is None or kv is not None:
                raise RuntimeError("context parallel forward needs enable_context_parallel and no KV cache")
            if T > self.cp.max_tokens:
                raise ValueError(f"{T} local tokens exceed the context-parallel buffers ({self.cp.max_tokens})")
            cp_geom = (nseq, cp_seq_len)
            pos.copy_(self.cp.local_positions(cp_seq_len).to(device=self.dev, dtype=torch.int32).repeat(nseq))
            tiles = None
        else:
            pos.copy_(torch.arange(S, device=self.dev, dtype=torch.int32).repeat(nseq))
            tiles, _ = self._tiles_for(nseq, S)
        res = None
        if self.first_stage:
            x = ws.get(f"{tag}.embed", (T, H))
            nv.embedding_fwd(tokens.reshape(-1), self.p.w["embed"], x, self.p.vocab_start)
            self.ctx.tp_all_reduce_(x)
        else:
            x, res = stage_in
        if kv is not None:
            slot = ws.get(f"{tag}.slot", (T,), torch.int32)
            slot.copy_((torch.arange(nseq, device=self.dev, dtype=torch.int32) * kv.max_len)
                       .repeat_interleave(S) + pos)
        for l in range(self.l0, self.l1):
            if kv is not None:
                # prefill: K/V go to the cache; attention reads them back from there
                ptiles = self._prefill_tiles(nseq, S, kv.max_len)
                x, res = self._layer_fwd(l, x, res, T, pos, tiles=ptiles, kbuf=kv.k[l], vbuf=kv.v[l],
                                         kv_slot=slot, tag=tag)
            else:
                if cp_geom is not None:
                    kb, vb = self.cp.bufs.local("k")[:T], self.cp.bufs.local("v")[:T]
                else:
                    kb = ws.get(f"{tag}.k", (T, self.p.kv_local))
                    vb = ws.get(f"{tag}.v", (T, self.p.kv_local))
                s_out = save.ckpt[l - self.l0] if save is not None else None
                if save is not None and res is None:
                    save.ckpt[0].copy_(x)          # the embedding output is layer 0's residual stream
                    x = save.ckpt[0]
                keep, stag, lse_l = None, None, None
                if save is not None and save.extra.get("stored"):
                    # keep this layer's expensive intermediates for its backward (no recompute)
                    stag = f"act{l - self.l0}"
                    kb = ws.get(f"{stag}.k", (T, self.p.kv_local))
                    vb = ws.get(f"{stag}.v", (T, self.p.kv_local))
                    lse_l = ws.get(f"{stag}.lse", (T, self.hq), torch.float32)
                    keep = {"k": kb, "v": vb, "lse": lse_l}
                    save.extra["keeps"].append(keep)
                x, res = self._layer_fwd(l, x, res, T, pos, tiles=tiles, kbuf=kb, vbuf=vb, lse=lse_l, keep=keep,
                                         s_in_out=s_out if res is not None else None, tag=tag, cp_geom=cp_geom,
                                         store_tag=stag)
        if not self.last_stage:
            return x, res
        hf = ws.get(f"{tag}.hf", (T, H))
        s_fin = ws.get(f"{tag}.s_fin", (T, H))
        nv.rmsnorm_fwd(x, self.p.w["norm"], hf, self.spec.rms_norm_eps, res=res, res_out=s_fin)
        if save is not None:
            save.final_s = s_fin
        return hf

    def _prefill_tiles(self, nseq: int, S: int, max_len: int):
        key = ("prefill", nseq, S, max_len)
        if key not in self._tiles:
            fw, _ = train_tiles(nseq, S, self.hq, self.hkv, self.d, self.dev)
            fw = fw.clone()
            b = torch.div(fw[:, 3], S, rounding_mode="floor")
            fw[:, 3] = b * max_len          # kv_row0 inside the cache
            self._tiles[key] = (fw.contiguous(), None)
        return self._tiles[key][0]

    # -------------------------------------------------------------------------- log-probs
    def logp_from_hidden(self, hf: torch.Tensor, targets: torch.Tensor, *, temperature: float = 1.0,
                         chunk: int = 8192, want_lse: bool = False, min_keep: torch.Tensor | None = None):
        """Selected-token log-prob of ``targets`` [R] from final hidden rows ``hf`` [R, H] through the
        fused LM-head epilogue; the [R, V] logits are never written.  ``min_keep`` [R] fp32 restricts the
        softmax of every row to the scaled logits at or above its value: the support the sampler drew from
        under top-k / top-p."""
        R = hf.shape[0]
        ntile = self.spec.num_vocab_tiles
        logp = torch.empty(R, dtype=torch.float32, device=self.dev)
        lse = torch.empty(R, dtype=torch.float32, device=self.dev) if want_lse else None
        for r0 in range(0, R, chunk):
            r1 = min(R, r0 + chunk)
            stats, tl = self._lmhead_stats(hf[r0:r1], targets[r0:r1], temperature, None,
                                           None if min_keep is None else min_keep[r0:r1])
            nv.logp_merge(stats, tl, logp[r0:r1], lse[r0:r1] if want_lse else None)
        return (logp, lse) if want_lse else logp

    def _lmhead_stats(self, hrows, targets, temperature, logits_out, min_keep=None):
        n = hrows.shape[0]
        ntile = self.spec.num_vocab_tiles
        tp = self.ctx.tp_size
        if tp > 1 and logits_out is None and hasattr(self.ctx.collective, "frame_tensor"):
            return self._lmhead_stats_fused_exchange(hrows, targets, temperature, min_keep)
        stats = self.ws.get("lm.stats", (n, ntile, 2), torch.float32)
        tl = self.ws.get("lm.tl", (n,), torch.float32)
        if tp > 1:
            stats.fill_(float("-inf"))
            stats[..., 1] = 0
            tl.zero_()
        w = self.p.w["lm_head"][: self.p.v_real_local] if self.p.v_real_local < self.p.v_local else self.p.w["lm_head"]
        if self.p.v_real_local < self.p.v_local:
            # tiles that are entirely padding keep (-inf, 0)
            stats[:, (self.p.vocab_start + self.p.v_real_local + VOCAB_TILE - 1) // VOCAB_TILE:] = \
                torch.tensor([float("-inf"), 0.0], device=self.dev)
        if self.p.v_real_local > 0:
            nv.lmhead_logp_stats(hrows, w, targets, stats, tl, vocab_start=self.p.vocab_start,
                                 inv_temp=1.0 / temperature, logits_out=logits_out, min_keep=min_keep)
        if tp > 1:
            # every rank filled only its own tiles / target: combine (exact: disjoint support)
            per = ntile // tp
            g = self.ctx.tp_all_gather(stats[:, self.ctx.tp_rank * per:(self.ctx.tp_rank + 1) * per].contiguous())
            stats = g.permute(1, 0, 2, 3).reshape(n, ntile, 2).contiguous()
            tl = self.ctx.tp_all_gather(tl).sum(0)
        return stats, tl

    LM_EXCHANGE_ROWS = 8192

    def _lmhead_stats_fused_exchange(self, hrows, targets, temperature, min_keep=None):
        """Vocab-parallel LM head with the statistics exchange inside the GEMM: every rank's epilogue
        stores its tiles' (max, sum-exp) and, for the rows whose target it owns, the target logit
        straight into all ranks' buffers over NVLink; one barrier later every rank merges complete
        rows locally.  Two buffer sets alternate so that a rank may start the next chunk while a
        peer still merges the previous one."""
        n = hrows.shape[0]
        ntile = self.spec.num_vocab_tiles
        if n > self.LM_EXCHANGE_ROWS:
            raise ValueError(f"at most {self.LM_EXCHANGE_ROWS} rows per LM-head call")
        if getattr(self, "_lm_peer", None) is None:
            from rl_kernel_b200.distributed.cp_attention import PeerMappedBuffers

            R = self.LM_EXCHANGE_ROWS
            specs = {}
            for q in (0, 1):
                specs[f"stats{q}"] = ((R, ntile, 2), torch.float32)
                specs[f"tl{q}"] = ((R,), torch.float32)
            self._lm_peer = PeerMappedBuffers(self.ctx.collective.group, self.dev, specs)
            for q in (0, 1):                             # tiles nobody owns (vocab padding) stay (-inf, 0)
                st = self._lm_peer.local(f"stats{q}")
                st[..., 0] = float("-inf")
                st[..., 1] = 0
            self._lm_parity = 0
            torch.cuda.synchronize(self.dev)
            self.ctx.collective.barrier()
        q = self._lm_parity
        self._lm_parity ^= 1
        pm = self._lm_peer
        w = self.p.w["lm_head"][: self.p.v_real_local]
        if self.p.v_real_local > 0:
            nv.lmhead_logp_stats_vp(hrows, w, targets, pm[f"stats{q}"], pm[f"tl{q}"], self.ctx.tp_rank,
                                    vocab_start=self.p.vocab_start, inv_temp=1.0 / temperature, min_keep=min_keep)
        self.ctx.collective.barrier()
        return pm.local(f"stats{q}")[:n], pm.local(f"tl{q}")[:n]

    # -------------------------------------------------------------------------- training step pieces
    def new_train_state(self, nseq: int, S: int, slot: int = 0) -> TrainState:
        """``slot`` separates the checkpoints of micro-batches that are in flight at the same time
        (pipeline schedules)."""
        T, H, L = nseq * S, self.spec.hidden_size, self.l1 - self.l0
        return TrainState(nseq, S, self.ws.get("ckpt" if slot == 0 else f"ckpt{slot}", (L, T, H)))

    def response_index(self, S: int, resp_start: int) -> tuple[torch.Tensor, torch.Tensor]:
        """(local row of every scored position this rank holds, its response index).  Position t
        scores token t+1, so the scored positions are resp_start-1 .. S-2; without context
        parallelism every rank holds all of them."""
        if self.cp is None:
            sel = torch.arange(resp_start - 1, S - 1, device=self.dev)
            return sel, sel + 1 - resp_start
        lpos = self.cp.local_positions(S).to(self.dev)
        sel = torch.nonzero((lpos >= resp_start - 1) & (lpos <= S - 2)).reshape(-1)
        return sel, lpos[sel] + 1 - resp_start

    def local_tokens(self, tokens: torch.Tensor) -> torch.Tensor:
        """The columns of ``tokens`` [nseq, S] this context-parallel rank holds (all without CP)."""
        if self.cp is None:
            return tokens
        return tokens[:, self.cp.local_positions(tokens.shape[1]).to(self.dev)].contiguous()

    def train_forward_backward(self, tokens: torch.Tensor, resp_start: int, dlogp_fn, *,
                               temperature: float = 1.0, lm_chunk: int = 4096, stage_in=None,
                               store_activations: bool = False, min_keep: torch.Tensor | None = None):
        """One micro-batch: forward with checkpoints, LM head + log-probs on response positions,
        ``dlogp_fn(logp [nseq, Rl]) -> dlogp [nseq, Rl]`` supplies d(loss)/d(logp), then the full
        backward accumulates into ``params.grad``.  Returns logp [nseq, Rl] (fp32).

        Position t predicts token t+1; response tokens are ``tokens[:, resp_start:]``, so positions
        ``resp_start-1 .. S-2`` are scored.  ``tokens`` is always the full [nseq, S] matrix; with
        context parallelism this rank embeds and scores only its own positions and the Rl columns
        of logp are the response indices ``response_index(S, resp_start)[1]``.
        ``min_keep`` [nseq, S - resp_start] fp32: the rollout's per-token sampling-support threshold (top-k /
        top-p); the log-prob and its gradient are then those of the distribution restricted to that support.
        """
        nseq, S = tokens.shape
        H = self.spec.hidden_size
        cp = self.cp is not None
        tok_local = self.local_tokens(tokens)
        Sl = tok_local.shape[1]
        sel, ridx = self.response_index(S, resp_start)
        R = sel.numel()
        st = self.new_train_state(nseq, Sl)
        st.extra["S_global"] = S
        if store_activations and not cp and self.supports_stored_activations:
            # trade memory for time: backward reuses the forward's tensors instead of recomputing
            # every layer (about 100 KB per token and layer at Qwen3-8B width)
            st.extra["stored"], st.extra["keeps"] = True, []
        hf = self.forward_hidden(tok_local, save=st, cp_seq_len=S if cp else None, stage_in=stage_in)
        if self._cp_canon:
            logp_local, dhf = self._head_cp_canonical(hf, tokens, resp_start, dlogp_fn, temperature, lm_chunk, sel, ridx,
                                                      min_keep)
            self.stage_input_grad = self._backward(st, tok_local, dhf)
            return logp_local
        hf3 = hf.view(nseq, Sl, H)
        rows = self.ws.get("lm.rows", (nseq * R, H))
        if cp:
            torch.index_select(hf3, 1, sel, out=rows.view(nseq, R, H))
        else:
            rows.view(nseq, R, H).copy_(hf3[:, resp_start - 1:S - 1])
        targets = tokens[:, resp_start:][:, ridx].reshape(-1).contiguous() if cp else \
            tokens[:, resp_start:].reshape(-1).contiguous()
        keep = None
        if min_keep is not None:
            keep = (min_keep[:, ridx] if cp else min_keep).reshape(-1).float().contiguous()
        # ---- pass 1: log-probs (fused stats).  A single-chunk, single-shard head keeps the bf16
        # logits the same kernel can write, so pass 2 does not have to multiply again.
        vloc = self.p.v_real_local
        # the logits buffer spans the padded shard: the canonical input-gradient GEMM runs over equal
        # vocabulary chunks, the padding columns stay zero (their weights are zero as well)
        vpad = self.p.v_local if self.canonical_grads else vloc
        lbuf = self.ws.get("lm.logits", (lm_chunk, vpad))
        if vpad > vloc:
            lbuf[:, vloc:].zero_()      # (the buffer may share memory with the rollout's KV cache)
        kept_logits = None
        if self.ctx.tp_size == 1 and nseq * R <= lm_chunk and vloc > 0:
            kept_logits = lbuf[: nseq * R, :vloc]
            stats, tl = self._lmhead_stats(rows, targets, temperature, kept_logits, keep)
            logp = torch.empty(nseq * R, dtype=torch.float32, device=self.dev)
            lse = torch.empty(nseq * R, dtype=torch.float32, device=self.dev)
            nv.logp_merge(stats, tl, logp, lse)
        else:
            logp, lse = self.logp_from_hidden(rows, targets, temperature=temperature, want_lse=True, min_keep=keep)
        dlogp = dlogp_fn(logp.view(nseq, R)).reshape(-1).contiguous()
        # ---- pass 2: per chunk, logits -> dlogits -> dH, dW
        drows = self.ws.get("lm.drows", (nseq * R, H))
        wlm = self.p.w["lm_head"][:vloc]
        glm = self.p.g["lm_head"][:vloc]
        for r0 in range(0, nseq * R, lm_chunk):
            r1 = min(nseq * R, r0 + lm_chunk)
            n = r1 - r0
            logits = lbuf[:n, :vloc]
            if vloc > 0:
                if kept_logits is None:
                    self._gemm(rows[r0:r1], wlm, logits)
                nv.dlogits_(logits, targets[r0:r1], lse[r0:r1], dlogp[r0:r1],
                            vocab_start=self.p.vocab_start, inv_temp=1.0 / temperature,
                            min_keep=None if keep is None else keep[r0:r1])
                if self.canonical_grads:
                    self._gemm(lbuf[:n], self.p.w["lm_head"], drows[r0:r1], b_mn=True, nchunks=self.nchunks,
                               M=n, N=H, K=vpad)
                else:
                    self._gemm(logits, wlm, drows[r0:r1], b_mn=True, M=n, N=H, K=vloc)
                self._gemm(logits, rows[r0:r1], glm, a_mn=True, b_mn=True, accumulate=True,
                           M=vloc, N=H, K=n)
            else:
                drows[r0:r1].zero_()
        self.ctx.tp_all_reduce_(drows)
        dhf = self.ws.get("b.dhf", (nseq * Sl, H))
        dhf.zero_()
        if cp:
            dhf.view(nseq, Sl, H).index_copy_(1, sel, drows.view(nseq, R, H))
        else:
            dhf.view(nseq, Sl, H)[:, resp_start - 1:S - 1].copy_(drows.view(nseq, R, H))
        self.stage_input_grad = self._backward(st, tok_local, dhf)   # None unless a pipeline stage
        return logp.view(nseq, R)

    def _head_cp_canonical(self, hf, tokens, resp_start: int, dlogp_fn, temperature: float, lm_chunk: int, sel, ridx,
                           min_keep=None):
        """LM head of a context-parallel micro-batch with layout-invariant results.

        The final hidden rows of ALL ranks are gathered into logical order, so the head sees exactly the rows a single
        GPU would; the vocabulary shard of this tensor-parallel rank is split once more over the CP ranks, and every
        rank computes the statistics, d(logits) and the weight-gradient rows of its slice for all rows.  Tile
        statistics are exchanged unchanged and merged in ascending tile order; the input gradient sums the canonical
        vocabulary chunks in the fixed tree (inside the kernel, then over the CP group, then over the TP group).
        Returns (logp [nseq, R_local] of this rank's scored positions, d(final hidden) [nseq * S_local, H])."""
        nseq, S = tokens.shape
        H, ws = self.spec.hidden_size, self.ws
        cpc, cp, c = self.ctx.cp_collective, self.ctx.cp_size, self.ctx.cp_rank
        Sl = S // cp
        R = S - resp_start
        n = nseq * R
        inv_t = 1.0 / temperature
        hf_g = self._cp_gather(hf, "cpg.hf", (nseq, S)).view(nseq, S, H)
        rows = ws.get("lm.rows_g", (n, H))
        rows.view(nseq, R, H).copy_(hf_g[:, resp_start - 1:S - 1])
        targets = tokens[:, resp_start:].reshape(-1).contiguous()
        keep = None if min_keep is None else min_keep.reshape(-1).float().contiguous()
        # ---- this rank's vocabulary slice of the TP shard
        if self.p.v_local % (cp * VOCAB_TILE) or self.nchunks % cp:
            raise ValueError(f"canonical context-parallel LM head: the vocabulary shard ({self.p.v_local} ids, "
                             f"{self.nchunks} canonical chunks on this tensor-parallel rank) must split into cp = {cp} "
                             "slices of whole 128-id tiles and whole chunks (tp x cp <= canonical_tp)")
        vs = self.p.v_local // cp
        v0 = c * vs
        vreal = max(0, min(vs, self.p.v_real_local - v0))
        gstart = self.p.vocab_start + v0                       # first global id of the slice
        w_slice = self.p.w["lm_head"][v0:v0 + vs]
        g_slice = self.p.g["lm_head"][v0:v0 + vs]
        nch = self.nchunks // cp
        ntile, nts = self.spec.num_vocab_tiles, vs // VOCAB_TILE
        logp = torch.empty(n, dtype=torch.float32, device=self.dev)
        lse = torch.empty(n, dtype=torch.float32, device=self.dev)
        # ---- pass 1: tile statistics of the slice, exchanged over CP and TP, merged in tile order
        for r0 in range(0, n, lm_chunk):
            r1 = min(n, r0 + lm_chunk)
            m = r1 - r0
            stats = ws.get("lm.stats_s", (m, nts, 2), torch.float32)
            stats[..., 0] = float("-inf")
            stats[..., 1] = 0
            tl = ws.get("lm.tl_s", (m,), torch.float32)
            tl.zero_()
            if vreal > 0:
                # the kernel indexes tiles globally: hand it a view that starts at tile 0 of this slice
                full = ws.get("lm.stats_f", (m, ntile, 2), torch.float32)
                nv.lmhead_logp_stats(rows[r0:r1], w_slice[:vreal], targets[r0:r1], full, tl, vocab_start=gstart,
                                     inv_temp=inv_t, min_keep=None if keep is None else keep[r0:r1])
                t0 = gstart // VOCAB_TILE
                nlive = (vreal + VOCAB_TILE - 1) // VOCAB_TILE
                stats[:, :nlive] = full[:, t0:t0 + nlive]
            shard = cpc.all_gather(stats).permute(1, 0, 2, 3).reshape(m, cp * nts, 2)        # this TP shard's tiles
            tls = cpc.all_gather(tl).sum(0)
            if self.ctx.tp_size > 1:
                shard = self.ctx.tp_all_gather(shard.contiguous()).permute(1, 0, 2, 3).reshape(m, ntile, 2)
                tls = self.ctx.tp_all_gather(tls).sum(0)
            nv.logp_merge(shard.contiguous(), tls.contiguous(), logp[r0:r1], lse[r0:r1])
        logp_local = logp.view(nseq, R)[:, ridx].contiguous()
        dlogp_local = dlogp_fn(logp_local)
        dlogp = torch.zeros(nseq, R, dtype=torch.float32, device=self.dev)
        dlogp[:, ridx] = dlogp_local.float()
        cpc.all_reduce_(dlogp)                                   # every column has one owner: exact
        dlogp = dlogp.reshape(-1)
        # ---- pass 2: logits of the slice -> d(logits) -> d(rows) (canonical chunks), dW rows of the slice
        drows = ws.get("lm.drows_g", (n, H))
        lbuf = ws.get("lm.logits_s", (min(n, lm_chunk), vs))
        if vreal < vs:
            lbuf[:, vreal:].zero_()
        for r0 in range(0, n, lm_chunk):
            r1 = min(n, r0 + lm_chunk)
            m = r1 - r0
            if vreal > 0:
                logits = lbuf[:m, :vreal]
                self._gemm(rows[r0:r1], w_slice[:vreal], logits)
                nv.dlogits_(logits, targets[r0:r1], lse[r0:r1], dlogp[r0:r1], vocab_start=gstart, inv_temp=inv_t,
                            min_keep=None if keep is None else keep[r0:r1])
                self._gemm(lbuf[:m], w_slice, drows[r0:r1], b_mn=True, nchunks=nch, M=m, N=H, K=vs)
                self._gemm(logits, rows[r0:r1], g_slice[:vreal], a_mn=True, b_mn=True, accumulate=True, M=vreal, N=H, K=m)
            else:
                drows[r0:r1].zero_()
        cpc.all_reduce_(drows)
        self.ctx.tp_all_reduce_(drows)
        dhf = ws.get("b.dhf", (nseq * Sl, H))
        dhf.zero_()
        dhf.view(nseq, Sl, H).index_copy_(1, sel, drows.view(nseq, R, H)[:, ridx])
        return logp_local, dhf

    def _backward(self, st: TrainState, tokens: torch.Tensor, dhf: torch.Tensor | None,
                  ds_in: torch.Tensor | None = None) -> torch.Tensor | None:
        """Backward of this stage's layers.  Last stage: ``dhf`` is the gradient of the final-norm
        output.  Other stages: ``ds_in`` is the gradient of the residual stream after the stage's last
        layer (what the next stage returned).  Returns the gradient of the stage input's residual
        stream for the previous stage (None on the first stage, which ends in the embedding)."""
        spec, w, g, ws = self.spec, self.p.w, self.p.g, self.ws
        nseq, S = st.nseq, st.S
        T, H = nseq * S, spec.hidden_size
        eps = spec.rms_norm_eps
        pos = ws.get("pos", (T,), torch.int32)
        cp = self.cp is not None
        cp_geom = (nseq, st.extra["S_global"]) if cp else None
        tiles, kvtiles = (None, None) if cp else self._tiles_for(nseq, S)
        scr = ws.get("b.scr", (max(nv.rmsnorm_bwd_scratch_elems(T, H), nv.qk_norm_rope_bwd_scratch_elems(T)),),
                     torch.float32)
        ds = ws.get("b.ds", (T, H))          # gradient of the residual stream
        cg = cp_geom if self._cp_canon else None
        if self.last_stage:
            # final norm: s_fin -> hf
            self._gain_bwd(st.final_s, w["norm"], dhf, ds, scr, eps, g["norm"], owner=0, cp_geom=cg)
        else:
            ds.copy_(ds_in)
        if cg is not None and self.ctx.tp_size > 1 and self.l1 > self.l0:
            self._qk_stage().zero_()                 # only the owner of a layer writes its row
        if cp:
            # peers read these while computing their dK / dV
            lse, delta = self.cp.bufs.local("lse"), self.cp.bufs.local("delta")
        else:
            lse = ws.get("b.lse", (T, self.hq), torch.float32)
            delta = ws.get("b.delta", (T, self.hq), torch.float32)
        for l in range(self.l1 - 1, self.l0 - 1, -1):
            keep: dict = {}
            ck = st.ckpt[l - self.l0]
            if cp:
                kb, vb = self.cp.bufs.local("k")[:T], self.cp.bufs.local("v")[:T]
            else:
                kb = ws.get("f.k", (T, self.p.kv_local))
                vb = ws.get("f.v", (T, self.p.kv_local))
            if st.extra.get("stored"):
                # the forward kept qkv, q, k, v, attention output, s_mid, gate/up and lse of this layer;
                # the two norms and the activation are rebuilt (bitwise the forward's values)
                keep = dict(st.extra["keeps"][l - self.l0])
                kb, vb, lse = keep["k"], keep["v"], keep["lse"]
                keep["h"] = ws.get("r.h", (T, H))
                nv.rmsnorm_fwd(ck, w[f"l{l}.ln1"], keep["h"], eps)
                keep["h2"] = ws.get("r.h2", (T, H))
                nv.rmsnorm_fwd(keep["s_mid"], w[f"l{l}.ln2"], keep["h2"], eps)
                self._rebuild_mlp_activation(keep, T)
            else:
                # ---- recompute the layer from its checkpointed input
                self._layer_fwd(l, ck, None, T, pos, tiles=tiles, kbuf=kb, vbuf=vb, lse=lse,
                                keep=keep, tag="r", cp_geom=cp_geom)
            # ---- MLP backward.  s_out = s_mid + down  =>  d(down) = ds, d(s_mid) += ds
            dh2 = self._mlp_bwd(l, ds, keep, T, cg)
            ds2 = ws.get("b.ds2", (T, H))
            self._gain_bwd(keep["s_mid"], w[f"l{l}.ln2"], dh2, ds2, scr, eps, g[f"l{l}.ln2"], dres=ds,
                           owner=2 * l + 1, cp_geom=cg)
            # ---- attention block backward.  s_mid = s_in + o  =>  d(o) = ds2
            dattn = self.cp.bufs.local("do")[:T] if cp else ws.get("b.dattn", (T, self.p.q_local))
            self._gemm(ds2, w[f"l{l}.wo"], dattn, b_mn=True, M=T, N=self.p.q_local, K=H)
            self._dw(ds2, keep["attn"], g[f"l{l}.wo"], M=H, N=self.p.q_local, T=T, cp_geom=cg)
            nv.attn_bwd_delta(keep["attn"], dattn, delta, T, self.hq)
            dq = ws.get("b.dq", (T, self.p.q_local))
            dk = ws.get("b.dk", (T, self.p.kv_local))
            dv = ws.get("b.dv", (T, self.p.kv_local))
            if cp:
                self.cp.backward_inplace(dq, dk, dv, *cp_geom)
            else:
                nv.attn_bwd_dq(keep["q"], dattn, kb, vb, lse, delta, dq, tiles, self.scale)
                nv.attn_bwd_dkv(keep["q"], dattn, kb, vb, lse, delta, dk, dv, kvtiles, self.scale)
            dqkv = ws.get("b.dqkv", (T, self.p.qkv_local))
            if self.canonical_grads:
                tp = self.ctx.tp_size
                # single rank: straight into the gradient (q_norm and k_norm gains are adjacent slots);
                # tensor parallel: a per-layer stage that is all-reduced once per micro-batch
                dqk = self._qk_grad_view()[l - self.l0] if tp == 1 else self._qk_stage()[l - self.l0]
                if cg is None:
                    nv.qk_norm_rope_bwd_canonical(keep["qkv"], w[f"l{l}.qn"], w[f"l{l}.kn"], self.cos, self.sin, pos,
                                                  dq, dk, dv, dqkv, scr, dqk, Hq=self.hq, Hkv=self.hkv, eps=eps,
                                                  accumulate_dw=tp == 1)
                else:
                    # this rank's rows give dqkv; the gain gradients come from all tokens in logical order,
                    # evaluated by the layer's owner rank
                    nv.qk_norm_rope_bwd_canonical(keep["qkv"], w[f"l{l}.qn"], w[f"l{l}.kn"], self.cos, self.sin, pos,
                                                  dq, dk, dv, dqkv, scr, ws.get("cpg.dqk_dummy", (256,)), Hq=self.hq,
                                                  Hkv=self.hkv, eps=eps, accumulate_dw=False)
                    qkv_g = self._cp_gather(keep["qkv"], "cpg.qkv", cg)
                    dq_g = self._cp_gather(dq, "cpg.dq", cg)
                    dk_g = self._cp_gather(dk, "cpg.dk", cg)
                    dv_g = self._cp_gather(dv, "cpg.dv", cg)
                    if l % self.ctx.cp_size == self.ctx.cp_rank:
                        Tg = qkv_g.shape[0]
                        pos_g = ws.get("cpg.pos", (Tg,), torch.int32)
                        pos_g.view(cg[0], cg[1]).copy_(torch.arange(cg[1], device=self.dev, dtype=torch.int32))
                        scr_g = ws.get("cpg.qscr", (nv.qk_norm_rope_bwd_scratch_elems(Tg),), torch.float32)
                        nv.qk_norm_rope_bwd_canonical(qkv_g, w[f"l{l}.qn"], w[f"l{l}.kn"], self.cos, self.sin, pos_g,
                                                      dq_g, dk_g, dv_g, ws.get("cpg.dqkv", (Tg, self.p.qkv_local)), scr_g,
                                                      dqk, Hq=self.hq, Hkv=self.hkv, eps=eps, accumulate_dw=tp == 1)
            else:
                nv.qk_norm_rope_bwd(keep["qkv"], w[f"l{l}.qn"], w[f"l{l}.kn"], self.cos, self.sin, pos,
                                    dq, dk, dv, dqkv, scr, g[f"l{l}.qn"], g[f"l{l}.kn"], Hq=self.hq,
                                    Hkv=self.hkv, eps=eps, accumulate_dw=True)
            dh = ws.get("b.dh", (T, H))
            self._gemm(dqkv, w[f"l{l}.wqkv"], dh, b_mn=True, nchunks=self.nchunks, M=T, N=H,
                       K=self.p.qkv_local)
            self.ctx.tp_all_reduce_(dh)
            self._dw(dqkv, keep["h"], g[f"l{l}.wqkv"], M=self.p.qkv_local, N=H, T=T, cp_geom=cg)
            self._gain_bwd(ck, w[f"l{l}.ln1"], dh, ds, scr, eps, g[f"l{l}.ln1"], dres=ds2, owner=2 * l, cp_geom=cg)
        if self.canonical_grads and self.ctx.tp_size > 1 and self.l1 > self.l0:
            # finish the KV-group tree over the tensor-parallel ranks, then accumulate
            st_qk = self._qk_stage()
            self.ctx.collective.all_reduce_(st_qk)
            self._qk_grad_view().add_(st_qk)
        if not self.first_stage:
            return ds
        # ---- embedding
        if cg is not None:
            # all tokens in logical order on one owner rank (the other ranks contribute nothing)
            ds_g = self._cp_gather(ds, "cpg.ds", cg)
            ids_g = self._cp_gather(tokens.reshape(-1, 1).contiguous(), "cpg.ids", cg).reshape(-1)
            if self.ctx.cp_rank == 0:
                sid, order = torch.sort(ids_g, stable=True)
                nv.embedding_bwd(sid.contiguous(), order.contiguous(), ds_g, g["embed"], self.p.vocab_start)
            return None
        sid, order = torch.sort(tokens.reshape(-1), stable=True)
        nv.embedding_bwd(sid.contiguous(), order.contiguous(), ds, g["embed"], self.p.vocab_start)
        return None

    # -------------------------------------------------------------------------- pipeline stages
    def stage_forward(self, tokens: torch.Tensor, stage_in, slot: int = 0):
        """Forward of a stage that does not own the head: returns (TrainState, (x, res))."""
        nseq, S = tokens.shape
        st = self.new_train_state(nseq, S, slot)
        out = self.forward_hidden(tokens, save=st, stage_in=stage_in)
        return st, out

    def stage_backward(self, st: TrainState, tokens: torch.Tensor, ds_in: torch.Tensor):
        """Backward of a stage that does not own the head; returns the gradient for the previous
        stage (None on the first stage)."""
        # recompute needs this micro-batch's positions again (another one may have run in between)
        pos = self.ws.get("pos", (st.nseq * st.S,), torch.int32)
        pos.copy_(torch.arange(st.S, device=self.dev, dtype=torch.int32).repeat(st.nseq))
        return self._backward(st, tokens, None, ds_in)

    # -------------------------------------------------------------------------- rollout
    def kv_cache_bytes(self, nseq: int, max_len: int) -> int:
        return 2 * self.spec.num_hidden_layers * nseq * max_len * self.p.kv_local * 2

    def new_kv_cache(self, nseq: int, max_len: int, storage: torch.Tensor | None = None) -> KVCache:
        """K and V of every layer, zero-filled.  ``storage`` (uint8, at least ``kv_cache_bytes``)
        lets the caller place the cache in memory it also uses for something else at other times."""
        L = self.spec.num_hidden_layers
        n = nseq * max_len * self.p.kv_local
        if storage is None:
            storage = torch.zeros(self.kv_cache_bytes(nseq, max_len), dtype=torch.uint8, device=self.dev)
        flat = storage[: 2 * L * n * 2].view(BF16)
        flat.zero_()
        k = [flat[(2 * l) * n:(2 * l + 1) * n].view(nseq * max_len, self.p.kv_local) for l in range(L)]
        v = [flat[(2 * l + 1) * n:(2 * l + 2) * n].view(nseq * max_len, self.p.kv_local) for l in range(L)]
        return KVCache(k, v, nseq, max_len, flat)

    def shared_prefix_cache_bytes(self, num_prompts: int, group: int, prompt_len: int, resp_len: int) -> int:
        rows = num_prompts * prompt_len + num_prompts * group * ((resp_len + 127) // 128 * 128)
        return 2 * self.spec.num_hidden_layers * rows * self.p.kv_local * 2

    def new_shared_prefix_cache(self, num_prompts: int, group: int, prompt_len: int, resp_len: int,
                                storage: torch.Tensor | None = None) -> SharedPrefixKV:
        """Pool for ``num_prompts * group`` sequences whose first ``prompt_len`` keys (a multiple of
        128) are the group's shared prompt.  Nothing is copied per sample: a sequence's page table
        names the prompt's pages for its first blocks and its own pages after them."""
        if prompt_len % 128:
            raise ValueError("shared-prefix pages need a prompt length that is a multiple of 128")
        L, P = self.spec.num_hidden_layers, prompt_len
        rp = (resp_len + 127) // 128 * 128
        nseq = num_prompts * group
        rows = num_prompts * P + nseq * rp
        n = rows * self.p.kv_local
        if storage is None:
            storage = torch.zeros(2 * L * n * 2, dtype=torch.uint8, device=self.dev)
        if storage.numel() < 2 * L * n * 2:
            raise ValueError(f"storage holds {storage.numel()} bytes, the pool needs {2 * L * n * 2}")
        flat = storage[: 2 * L * n * 2].view(BF16)
        flat.zero_()
        k = [flat[(2 * l) * n:(2 * l + 1) * n].view(rows, self.p.kv_local) for l in range(L)]
        v = [flat[(2 * l + 1) * n:(2 * l + 2) * n].view(rows, self.p.kv_local) for l in range(L)]
        kv = KVCache(k, v, 1, rows, flat)
        pkv = KVCache([t[: num_prompts * P] for t in k], [t[: num_prompts * P] for t in v], num_prompts, P, None)
        b = torch.arange(nseq)
        pb, rb = P // 128, rp // 128
        prompt_pages = (b // group).view(-1, 1) * pb + torch.arange(pb).view(1, -1)
        own_pages = (num_prompts * P) // 128 + b.view(-1, 1) * rb + torch.arange(rb).view(1, -1)
        table = torch.cat([prompt_pages, own_pages], dim=1).to(torch.int32).to(self.dev).contiguous()
        slot_base = (num_prompts * P + b * rp).to(torch.int32).to(self.dev)
        return SharedPrefixKV(kv, pkv, table, slot_base, P, pb + rb)

    def decode_tiles_shared_prefix(self, sp: SharedPrefixKV, group: int) -> torch.Tensor:
        """Decode tiles for a shared-prefix pool, ordered (prompt, KV head, sample) so that the tiles
        that read the same prompt pages run next to each other and share them through L2."""
        nseq = sp.page_table.shape[0]
        t = self.decode_tiles(nseq, 0)
        b = torch.arange(nseq).view(-1, 1).expand(nseq, self.hkv).reshape(-1)
        t[:, 3] = 0
        t[:, 11] = (b * sp.blocks_per_seq + 1).to(torch.int32).to(self.dev)
        hk = torch.arange(self.hkv).view(1, -1).expand(nseq, self.hkv).reshape(-1)
        order = torch.argsort((b // group) * (self.hkv * group) + hk * group + b % group, stable=True)
        t = t[order.to(self.dev)].contiguous()
        g = self.hq // self.hkv
        P = sp.prompt_len
        if P % 128 == 0 and P > 0 and nseq % group == 0 and g * group <= 32 and (g * group) % 8 == 0:
            npr = nseq // group
            pi = torch.arange(npr).view(-1, 1).expand(npr, self.hkv).reshape(-1)
            ph = torch.arange(self.hkv).view(1, -1).expand(npr, self.hkv).reshape(-1)
            z = torch.zeros_like(pi)
            row0 = pi * group * self.hq + ph * g
            pt = torch.stack([row0, z, z + g * group, z, ph * self.d, z + P - 1, z, z + P, z, z + 1, z,
                              pi * group * sp.blocks_per_seq + 1], dim=-1)
            sp.prefix_tiles = pt.to(torch.int32).to(self.dev).contiguous()
            sp.prefix_ext = torch.stack([z, z + 1, row0, z], dim=-1).to(torch.int32).to(self.dev).contiguous()
            se = torch.zeros(t.shape[0], 4, dtype=torch.int32, device=self.dev)
            se[:, 0] = P // 128
            se[:, 1] = 2
            se[:, 2] = t[:, 0]
            sp.seq_ext = se.contiguous()
            sp.row_state = torch.zeros(nseq * self.hq, 136, dtype=torch.float32, device=self.dev)
            sp.group = group
        return t

    def decode_tiles(self, nseq: int, max_len: int) -> torch.Tensor:
        """Static part of the decode tile table; columns 5 (pos0) and 7 (kv_cap) change per step."""
        g = self.hq // self.hkv
        b = torch.arange(nseq).view(-1, 1)
        hk = torch.arange(self.hkv).view(1, -1)
        z = torch.zeros(nseq, self.hkv, dtype=torch.long)
        row0 = b * self.hq + hk * g + z
        t = torch.stack([row0, z, z + g, b * max_len + z, hk * self.d + z, z, z, z + 1, row0, z + 1, z, z],
                        dim=-1).reshape(-1, 12)
        return t.to(torch.int32).to(self.dev).contiguous()

    def decode_step(self, tokens: torch.Tensor, pos: torch.Tensor, kv: KVCache, tiles: torch.Tensor,
                    shared: SharedPrefixKV | None = None) -> torch.Tensor:
        """One token per sequence: tokens [B] at positions ``pos`` [B] (int32) -> final hidden [B, H].
        ``tiles`` comes from ``decode_tiles``; this call refreshes its position columns on the
        device, so the whole step can be captured in a CUDA graph.  ``shared``: the KV lives in a
        shared-prefix pool (``kv`` is ``shared.kv``, tiles from ``decode_tiles_shared_prefix``)."""
        B, H, L = tokens.shape[0], self.spec.hidden_size, self.spec.num_hidden_layers
        ws = self.ws
        slot = ws.get("d.slot", (B,), torch.int32)
        if shared is None:
            tiles[:, 5] = pos.repeat_interleave(self.hkv)
            torch.add(torch.arange(B, device=self.dev, dtype=torch.int32) * kv.max_len, pos, out=slot)
        else:
            # tiles are not in sequence order: column 0 (first query row) identifies the sequence
            if shared.seq_of_tile is None:
                shared.seq_of_tile = torch.div(tiles[:, 0], self.hq, rounding_mode="floor").long()
            tiles[:, 5] = pos[shared.seq_of_tile]
            torch.add(shared.slot_base, pos - shared.prompt_len, out=slot)
        tiles[:, 7] = tiles[:, 5] + 1
        self._decode_page_table = shared.page_table if shared is not None else None
        self._decode_shared = shared
        x = ws.get("d.embed", (B, H))
        nv.embedding_fwd(tokens, self.p.w["embed"], x, self.p.vocab_start)
        self.ctx.tp_all_reduce_(x)
        res = None
        for l in range(L):
            x, res = self._layer_fwd(l, x, res, B, pos, tiles=tiles, kbuf=kv.k[l], vbuf=kv.v[l],
                                     kv_slot=slot, q_view=(B * self.hq, self.d), tag="d")
        self._decode_page_table = None
        self._decode_shared = None
        hf = ws.get("d.hf", (B, H))
        s_fin = ws.get("d.s_fin", (B, H))
        self._norm_after(x, self.p.w["norm"], hf, res, s_fin)
        return hf

    def logits(self, hf: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """Local-vocab-shard logits [rows, v_real_local] (bf16)."""
        n = hf.shape[0]
        vloc = self.p.v_real_local
        if out is None:
            out = self.ws.get("d.logits", (n, vloc))
        with nv.static_weights():       # follows the final norm; the LM head is a weight
            self._gemm(hf, self.p.w["lm_head"][:vloc], out)
        return out

    def keep_threshold(self, logits: torch.Tensor, *, temperature: float, top_k: int = 0, top_p: float = 1.0):
        """Per-row smallest scaled logit that top-k / top-p keep (None when nothing is cut), from this rank's
        logits shard [n, V_local]; under tensor parallelism the shards are gathered first so that every rank
        derives the same threshold from the whole row."""
        if (not top_k or top_k <= 0) and top_p >= 1.0:
            return None
        n = logits.shape[0]
        vr = self.p.v_real_local
        rows = logits[:, :vr] if vr < logits.shape[1] else logits
        if self.ctx.tp_size > 1:
            full = self.ctx.tp_all_gather(logits.contiguous())                       # [tp, n, V_local]
            rows = full.permute(1, 0, 2).reshape(n, -1)[:, : self.spec.vocab_size].contiguous()
        thr = self.ws.get("s.thr", (n,), torch.float32)
        nv.sample_keep_threshold(rows if rows.stride(1) == 1 else rows.contiguous(), thr, inv_temp=1.0 / temperature,
                                 top_k=top_k, top_p=top_p)
        return thr

    def sample(self, logits: torch.Tensor, row_keys: torch.Tensor, *, temperature: float, seed: int,
               greedy: bool = False, top_k: int = 0, top_p: float = 1.0, return_threshold: bool = False):
        """Sample one id per row and return (ids, logp of the sampled id under the same temperature),
        the log-prob computed with the tile contract shared with the training path.  With ``top_k`` /
        ``top_p`` the draw and the log-prob are over the restricted support; ``return_threshold`` adds the
        per-row threshold that defines it (what the trainer replays as ``min_keep``)."""
        n = logits.shape[0]
        ids = self.ws.get("s.ids", (n,), torch.int64)
        val = self.ws.get("s.val", (n,), torch.float32)
        thr = self.keep_threshold(logits, temperature=temperature, top_k=top_k, top_p=top_p)
        nv.sample_gumbel(logits, ids, val, vocab_start=self.p.vocab_start, inv_temp=1.0 / temperature,
                         seed=seed, step=0, greedy=greedy, row_keys=row_keys, min_keep=thr)
        if self.ctx.tp_size > 1:
            vals = self.ctx.tp_all_gather(val)           # [tp, n]
            idss = self.ctx.tp_all_gather(ids)
            # the winner is the largest perturbed logit; among equal values the lowest rank wins (its
            # ids are the smallest), spelled out because argmax does not promise a tie order
            ranks = torch.arange(vals.shape[0], device=vals.device).view(-1, 1).expand_as(vals)
            best = torch.where(vals == vals.max(0, keepdim=True).values, ranks,
                               torch.full_like(ranks, vals.shape[0])).min(0, keepdim=True).values
            ids = idss.gather(0, best)[0].contiguous()
        ntile = self.spec.num_vocab_tiles
        stats = self.ws.get("s.stats", (n, ntile, 2), torch.float32)
        tl = self.ws.get("s.tl", (n,), torch.float32)
        stats[..., 0] = float("-inf")
        stats[..., 1] = 0
        tl.zero_()
        nv.logits_tile_stats(logits, ids, stats, tl, vocab_start=self.p.vocab_start,
                             inv_temp=1.0 / temperature, min_keep=thr)
        if self.ctx.tp_size > 1:
            per = ntile // self.ctx.tp_size
            gs = self.ctx.tp_all_gather(stats[:, self.ctx.tp_rank * per:(self.ctx.tp_rank + 1) * per].contiguous())
            stats = gs.permute(1, 0, 2, 3).reshape(n, ntile, 2).contiguous()
            tl = self.ctx.tp_all_gather(tl).sum(0)
        logp = self.ws.get("s.logp", (n,), torch.float32)
        nv.logp_merge(stats, tl, logp, None)
        if return_threshold:
            return ids, logp, thr
        return ids, logp
