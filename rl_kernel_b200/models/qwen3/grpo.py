"""A complete GRPO step on the sm_100a engine: weight publish -> rollout (prefill + CUDA-graph
decode with sampling) -> rewards/advantages -> reference log-probs -> training forward/backward
over micro-batches -> gradient clipping -> AdamW, plus the train-vs-rollout log-prob mismatch
counter that is the product's acceptance metric
(reports/archive/experiments/dense/convergence_s1234_g10_g11/README.md:16-24 in the reference).

The rollout engine and the trainer share the kernels but not the call pattern: rollout runs one
token per sequence against a KV cache, training runs packed full sequences; their selected-token
log-probs must be bitwise equal.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from rl_kernel_b200.backends import native as nv
from rl_kernel_b200.models.qwen3.engine import PackedParams, ParallelContext, Qwen3Engine
from rl_kernel_b200.models.qwen3.spec import Qwen3DenseSpec
from rl_kernel_b200.utils.bits import bit_mismatch_count


@dataclass
class GRPOConfig:
    num_prompts: int = 8
    group_size: int = 8
    prompt_len: int = 512
    response_len: int = 1024
    temperature: float = 1.0
    # sampling support of the rollout (0 / 1.0 = the whole vocabulary).  When either cuts the support, the
    # rollout records every token's keep threshold and reference scoring and training replay it, so
    # rollout and training log-probs are those of the same restricted distribution.
    top_k: int = 0
    top_p: float = 1.0
    clip_eps: float = 0.2
    kl_coef: float = 0.001
    lr: float = 1e-6
    beta1: float = 0.9
    beta2: float = 0.95
    adam_eps: float = 1e-8
    weight_decay: float = 0.01
    max_grad_norm: float = 1.0
    micro_batch_seqs: int = 8
    seed: int = 1234
    use_cuda_graph: bool = True
    use_reference_model: bool = True
    share_rollout_weights: bool = False   # True: rollout reads the trainer's buffer (zero-copy publish)
    # The rollout engine's own weight buffer lives in the memory of the gradient buffer: gradients
    # are dead between the optimizer step and the next backward, which is exactly when the rollout
    # runs.  Every step publishes with the weight-push kernel (csrc/collectives/weight_sync.cu).
    rollout_weights_in_grad_buffer: bool = False
    share_kv_and_activation_memory: bool = True
    share_prompt_pages: bool = True       # group members read their prompt's K/V pages in place
    store_activations: bool = False       # training keeps layer intermediates instead of recomputing them
    train_micro_batch_seqs: int = 0       # sequences per training micro-batch (0 = micro_batch_seqs)

    @property
    def num_seqs(self) -> int:
        return self.num_prompts * self.group_size

    @property
    def seq_len(self) -> int:
        return self.prompt_len + self.response_len

    @property
    def restricted_support(self) -> bool:
        return (self.top_k is not None and self.top_k > 0) or self.top_p < 1.0


class AdamW:
    """Fused AdamW over the flat parameter shard with fp32 master weights and exact,
    partition-independent gradient-norm clipping."""

    def __init__(self, params: PackedParams, cfg: GRPOConfig, ctx: ParallelContext):
        self.p, self.cfg, self.ctx = params, cfg, ctx
        n, dev = params.numel, params.device
        self.master = params.flat.float()
        self.m = torch.zeros(n, dtype=torch.float32, device=dev)
        self.v = torch.zeros(n, dtype=torch.float32, device=dev)
        self.bins = torch.zeros(256, dtype=torch.int64, device=dev)
        self.scale = torch.ones(1, dtype=torch.float32, device=dev)
        self.step_count = 0
        e = torch.arange(256, device=dev).clamp(min=1).double()
        self._bin_w = torch.pow(2.0, 2.0 * (e - 134.0))
        self._bin_w[255] = 0.0
        self.last_grad_norm = torch.zeros(1, dtype=torch.float64, device=dev)

    def grad_norm(self) -> torch.Tensor:
        """Exact global L2 norm of the bf16 gradient: integer bins per shard, integer all-reduce,
        one fixed-order fp64 combination.  Replicated parameters are counted once."""
        self.bins.zero_()
        if self.ctx.tp_size == 1:
            nv.sumsq_bins(self.p.grad, self.bins)
        else:
            for name, s in self.p.slots.items():
                if self.p.is_replicated(name) and self.ctx.tp_rank != 0:
                    continue
                nv.sumsq_bins(self.p.grad[s.offset:s.offset + s.numel], self.bins)
            self.ctx.collective.all_reduce_int_(self.bins)
        return (self.bins.double() * self._bin_w).sum().sqrt()

    def _sync_partial_replicated_grads(self) -> None:
        """q_norm / k_norm gains are replicated but each TP rank only saw its own heads: sum the
        partial gradients over TP (fixed tree) so every rank holds the same full gradient."""
        if self.ctx.tp_size == 1 or getattr(self.p, "qk_grads_complete", False):
            return                      # one rank, or the engine already finished the tree over the ranks
        names = [n for n in self.p.slots if n.endswith((".qn", ".kn"))]
        buf = torch.cat([self.p.g[n].reshape(-1) for n in names]).contiguous()
        self.ctx.collective.all_reduce_(buf)
        off = 0
        for n in names:
            k = self.p.g[n].numel()
            self.p.g[n].copy_(buf[off:off + k].view_as(self.p.g[n]))
            off += k

    def step(self) -> None:
        c = self.cfg
        self.step_count += 1
        self._sync_partial_replicated_grads()
        gn = self.grad_norm()
        self.last_grad_norm.copy_(gn.reshape(1))
        if c.max_grad_norm > 0:
            self.scale.copy_(torch.clamp(c.max_grad_norm / (gn + 1e-6), max=1.0).float().reshape(1))
        nv.adamw(self.master, self.m, self.v, self.p.grad, self.p.flat, lr=c.lr, beta1=c.beta1,
                 beta2=c.beta2, eps=c.adam_eps, weight_decay=c.weight_decay, step=self.step_count,
                 grad_scale=self.scale)


class GRPOTrainer:
    """Owns the policy (with gradients and optimizer), the frozen reference policy and the rollout
    state of one rank."""

    def __init__(self, spec: Qwen3DenseSpec, cfg: GRPOConfig, device: torch.device,
                 ctx: ParallelContext | None = None, weights=None):
        self.spec, self.cfg, self.dev = spec, cfg, device
        self.ctx = ctx or ParallelContext()
        tp_r, tp = self.ctx.tp_rank, self.ctx.tp_size
        # Context parallelism applies to training only.  For rollout the cp TP groups act as cp
        # independent engines, each generating for its share of the prompts.
        # Data parallelism: ``cfg.num_prompts`` counts the whole job; a replica (one TP x CP group)
        # rolls out and trains num_prompts / dp of them and the gradients are summed over replicas.
        self.cp, self.dp = self.ctx.cp_size, self.ctx.dp_size
        # sampling keys pack (global sequence, position) into the low 32 bits -- 16 bits each -- and
        # the training step into the high word; larger jobs would carry into the step's bits
        if cfg.num_seqs >= 65536 or cfg.seq_len > 65536:
            raise ValueError(f"sampling keys hold 65535 sequences x 65536 positions; got {cfg.num_seqs} x {cfg.seq_len}")
        if cfg.num_prompts % (self.cp * self.dp) or cfg.micro_batch_seqs < 1:
            raise ValueError(f"num_prompts {cfg.num_prompts} must be a multiple of cp x dp = {self.cp * self.dp}")
        self.rep_prompts = cfg.num_prompts // self.dp          # prompts of this replica
        self.rep_seqs = self.rep_prompts * cfg.group_size
        self.roll_prompts = self.rep_prompts // self.cp        # prompts of this rollout engine
        self.roll_seqs = self.roll_prompts * cfg.group_size
        self.engine_index = self.ctx.dp_rank * self.cp + self.ctx.cp_rank   # which rollout engine this is
        self.rollout_ctx = self.ctx if self.cp == 1 else ParallelContext(tp_r, tp, collective=self.ctx.collective)
        self.policy = PackedParams(spec, tp_r, tp, device, with_grad=True)
        if weights is not None:
            self.policy.load(weights)
        else:
            self.policy.init_synthetic_(cfg.seed)
        self.engine = Qwen3Engine(spec, self.policy, self.ctx, max_positions=cfg.seq_len + 8)
        self.policy.qk_grads_complete = self.engine.canonical_grads
        if self.cp > 1:
            self.engine.enable_context_parallel(cfg.micro_batch_seqs * cfg.seq_len // self.cp)
        self.ref_params = None
        if cfg.use_reference_model and cfg.kl_coef > 0:
            self.ref_params = PackedParams(spec, tp_r, tp, device)
            self.ref_params.flat.copy_(self.policy.flat)
        # rollout weights: a separate buffer that receives every published version, unless the
        # engines are colocated and configured to alias the trainer's shard
        self._push = None
        if cfg.share_rollout_weights:
            self.rollout_params = self.policy
        elif cfg.rollout_weights_in_grad_buffer:
            from rl_kernel_b200.integrations.common.weights import NVLinkPushBridge

            self.rollout_params = PackedParams(spec, tp_r, tp, device, storage=self.policy.grad)
            self._version_flag = torch.zeros(32, dtype=torch.int64, device=device)
            self._push = NVLinkPushBridge(self.policy, device, source_worker="trainer", source_rank=tp_r)
            self._push.add_target(self.rollout_params, version_flag_ptr=self._version_flag.data_ptr(), sole_writer=True)
            self._last_update_id = None
        else:
            self.rollout_params = PackedParams(spec, tp_r, tp, device)
        self.rollout_engine = Qwen3Engine(spec, self.rollout_params, self.rollout_ctx, max_positions=cfg.seq_len + 8)
        kv_bytes = self.rollout_engine.kv_cache_bytes(self.roll_seqs, cfg.seq_len)
        if cfg.share_prompt_pages and cfg.prompt_len % 128 == 0:
            kv_bytes = max(kv_bytes, self.rollout_engine.shared_prefix_cache_bytes(
                self.roll_prompts, cfg.group_size, cfg.prompt_len, cfg.response_len))
        self._arena = None
        if cfg.share_kv_and_activation_memory:
            self._arena = torch.zeros(kv_bytes, dtype=torch.uint8, device=device)
            self.engine.ws.arena = self._arena
        self.rollout_engine.ws = self.engine.ws      # rollout and training never overlap in time
        self.rollout_engine.cos, self.rollout_engine.sin = self.engine.cos, self.engine.sin
        self.weight_version = 0
        self.opt = AdamW(self.policy, cfg, self.ctx)
        self._graph = None
        self.graph_launches = 0
        self._kv = None
        self.metrics: dict[str, float] = {}

    def local_prompts(self, prompts: torch.Tensor) -> torch.Tensor:
        """The slice of the global prompt batch this rank's rollout engine generates for."""
        n = self.roll_prompts
        return prompts[self.engine_index * n:(self.engine_index + 1) * n]

    # ---------------------------------------------------------------- weight sync
    def publish_weights(self) -> int:
        """Train -> rollout weight sync with a monotonic version: the weight-push kernel when the
        trainer owns a push bridge, one device copy of the flat shard otherwise, nothing when the
        rollout engine aliases the trainer's buffer."""
        self.weight_version += 1
        if self._push is not None:
            m = self._push.publish(weight_version=self.weight_version)
            if self._last_update_id is not None:
                self._push.release(self._last_update_id)
            self._last_update_id = m.update_id
        elif self.rollout_params is not self.policy:
            self.rollout_params.flat.copy_(self.policy.flat)
        return self.weight_version

    # ---------------------------------------------------------------- rollout
    def _ensure_rollout_state(self):
        c = self.cfg
        if self._kv is None:
            B = self.roll_seqs
            eng = self.rollout_engine
            self._shared = None
            if c.share_prompt_pages and c.prompt_len % 128 == 0:
                self._shared = eng.new_shared_prefix_cache(self.roll_prompts, c.group_size, c.prompt_len,
                                                           c.response_len, storage=self._arena)
                self._kv, self._pkv = self._shared.kv, self._shared.prompt_kv
                self._dtiles = eng.decode_tiles_shared_prefix(self._shared, c.group_size)
            else:
                self._kv = eng.new_kv_cache(B, c.seq_len, storage=self._arena)
                self._pkv = eng.new_kv_cache(self.roll_prompts, c.prompt_len)
                self._dtiles = eng.decode_tiles(B, c.seq_len)
            self._tok = torch.zeros(B, dtype=torch.int64, device=self.dev)
            self._pos = torch.zeros(B, dtype=torch.int32, device=self.dev)
            self._keys = torch.zeros(B, dtype=torch.int64, device=self.dev)
            # sampling keys are global sequence numbers: the draw of a sequence does not depend on
            # which rollout engine generated it
            self._seq_key = (torch.arange(B, dtype=torch.int64, device=self.dev)
                             + self.engine_index * B) * 65536
            # the training step goes into the high word of the sampling keys through a device
            # tensor: a captured decode graph freezes scalar arguments such as the seed, and the
            # noise must still differ from one training step to the next
            self._step_key = torch.zeros(1, dtype=torch.int64, device=self.dev)
            self._out_tok = torch.zeros(B, c.response_len, dtype=torch.int64, device=self.dev)
            self._out_lp = torch.zeros(B, c.response_len, dtype=torch.float32, device=self.dev)
            self._out_thr = torch.zeros(B, c.response_len, dtype=torch.float32, device=self.dev) \
                if c.restricted_support else None
            self._col = torch.zeros(1, dtype=torch.int64, device=self.dev)

    def _decode_once(self):
        """tok[B] at pos[B] -> next token + its logp, appended at column `col`; advances state.
        (The training step reaches the sampler through ``_step_key``, not through an argument: this
        function is captured in a CUDA graph.)"""
        eng, c = self.rollout_engine, self.cfg
        hf = eng.decode_step(self._tok, self._pos, self._kv, self._dtiles, shared=self._shared)
        logits = eng.logits(hf)
        torch.add(self._seq_key, self._pos, out=self._keys)
        self._keys.add_(self._step_key)
        ids, lp, thr = eng.sample(logits, self._keys, temperature=c.temperature, seed=c.seed, top_k=c.top_k,
                                  top_p=c.top_p, return_threshold=True)
        col = self._col.expand(ids.shape[0]).unsqueeze(1)
        self._out_tok.scatter_(1, col, ids.unsqueeze(1))
        self._out_lp.scatter_(1, col, lp.unsqueeze(1))
        if thr is not None:
            self._out_thr.scatter_(1, col, thr.unsqueeze(1))
        self._tok.copy_(ids)
        self._pos.add_(1)
        self._col.add_(1)

    @torch.no_grad()
    def rollout(self, prompts: torch.Tensor, step_seed: int):
        """prompts [n, prompt_len] (this engine's share) -> (tokens [B, S], logp [B, R]); B = n x group."""
        c, eng = self.cfg, self.rollout_engine
        self._ensure_rollout_state()
        B, P, R, G = self.roll_seqs, c.prompt_len, c.response_len, c.group_size
        NP = self.roll_prompts
        if self._arena is not None:
            self._kv.flat.zero_()        # training activations lived here since the last rollout
        # ---- prefill each distinct prompt once, then share its KV with the whole group
        hf = eng.forward_hidden(prompts, kv=self._pkv, tag="p")
        H = self.spec.hidden_size
        last = hf.view(NP, P, H)[:, P - 1].repeat_interleave(G, dim=0).contiguous()
        if self._shared is None:
            for l in range(self.spec.num_hidden_layers):
                for src, dst in ((self._pkv.k[l], self._kv.k[l]), (self._pkv.v[l], self._kv.v[l])):
                    d3 = dst.view(NP, G, c.seq_len, -1)
                    d3[:, :, :P].copy_(src.view(NP, 1, P, -1).expand(-1, G, -1, -1))
        # ---- first response token comes from the prefill logits
        self._pos.fill_(P - 1)
        self._col.zero_()
        logits = eng.logits(last)
        self._step_key.fill_((int(step_seed) & 0x7FFFFFFF) << 32)
        torch.add(self._seq_key, self._pos, out=self._keys)
        self._keys.add_(self._step_key)
        ids, lp, thr = eng.sample(logits, self._keys, temperature=c.temperature, seed=c.seed, top_k=c.top_k,
                                  top_p=c.top_p, return_threshold=True)
        self._out_tok[:, 0].copy_(ids)
        self._out_lp[:, 0].copy_(lp)
        if thr is not None:
            self._out_thr[:, 0].copy_(thr)
        self._tok.copy_(ids)
        self._pos.fill_(P)
        self._col.fill_(1)
        # ---- decode R-1 more tokens
        if c.use_cuda_graph:
            if self._graph is None:
                # warm-up outside capture (allocations, attribute setting), then capture one step
                snap = (self._tok.clone(), self._pos.clone(), self._col.clone())
                s = torch.cuda.Stream(self.dev)
                s.wait_stream(torch.cuda.current_stream(self.dev))
                with torch.cuda.stream(s):
                    self._decode_once()
                torch.cuda.current_stream(self.dev).wait_stream(s)
                self._tok.copy_(snap[0]); self._pos.copy_(snap[1]); self._col.copy_(snap[2])
                self._graph = torch.cuda.CUDAGraph()
                n0 = nv.LAUNCH_COUNT
                coll = self.rollout_ctx.collective
                with torch.cuda.graph(self._graph):
                    if coll is not None:
                        with coll.graph_capture():
                            self._decode_once()
                    else:
                        self._decode_once()
                if coll is not None:
                    coll.graph_commit()
                self.graph_launches = nv.LAUNCH_COUNT - n0
                self._tok.copy_(snap[0]); self._pos.copy_(snap[1]); self._col.copy_(snap[2])
            for _ in range(R - 1):
                self._graph.replay()
            if self.rollout_ctx.collective is not None:
                self.rollout_ctx.collective.graph_replayed(R - 1)
            nv.LAUNCH_COUNT += (R - 1) * self.graph_launches
        else:
            for _ in range(R - 1):
                self._decode_once()
        tokens = torch.cat([prompts.repeat_interleave(G, dim=0), self._out_tok], dim=1).contiguous()
        self.last_support = self._out_thr.clone() if self._out_thr is not None else None
        return tokens, self._out_lp.clone()

    # ---------------------------------------------------------------- scoring with frozen weights
    @torch.no_grad()
    def score(self, params: PackedParams, tokens: torch.Tensor, min_keep: torch.Tensor | None = None) -> torch.Tensor:
        """Selected-token log-probs of the response tokens under ``params`` (no gradients):
        [n, Rl], the columns being this rank's response indices (all of them without CP)."""
        c = self.cfg
        eng = self.engine
        saved = eng.p
        eng.p = params
        S = c.seq_len
        sel, ridx = eng.response_index(S, c.prompt_len)
        try:
            out = []
            for b0 in range(0, tokens.shape[0], c.micro_batch_seqs):
                tk = tokens[b0:b0 + c.micro_batch_seqs]
                n = tk.shape[0]
                tl = eng.local_tokens(tk)
                hf = eng.forward_hidden(tl, cp_seq_len=S if self.cp > 1 else None).view(n, tl.shape[1], -1)
                rows = hf[:, sel].reshape(n * sel.numel(), -1).contiguous()
                mk = None if min_keep is None else min_keep[b0:b0 + c.micro_batch_seqs][:, ridx].reshape(-1).contiguous()
                lp = eng.logp_from_hidden(rows, tk[:, c.prompt_len:][:, ridx].reshape(-1).contiguous(),
                                          temperature=c.temperature, min_keep=mk)
                out.append(lp.view(n, sel.numel()).clone())
            return torch.cat(out)
        finally:
            eng.p = saved

    def _gather_rollouts(self, tokens: torch.Tensor, logp: torch.Tensor):
        """Every rollout engine's sequences, in global sequence order, on every rank."""
        if self.cp == 1:
            return tokens, logp
        import torch.distributed as dist

        tk = torch.empty((self.cp,) + tuple(tokens.shape), dtype=tokens.dtype, device=self.dev)
        lp = torch.empty((self.cp,) + tuple(logp.shape), dtype=logp.dtype, device=self.dev)
        dist.all_gather_into_tensor(tk, tokens.contiguous(), group=self.ctx.cp_group)
        dist.all_gather_into_tensor(lp, logp.contiguous(), group=self.ctx.cp_group)
        return tk.flatten(0, 1), lp.flatten(0, 1)

    # ---------------------------------------------------------------- one full step
    def step(self, prompts: torch.Tensor, rewards_fn=None, step_index: int = 0) -> dict:
        c = self.cfg
        B, R = self.rep_seqs, c.response_len          # sequences this replica trains on
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        ev[0].record()
        self.publish_weights()
        tokens, old_logp = self.rollout(prompts, step_seed=c.seed + 7919 * step_index)
        support = self.last_support                     # [B_engine, R] keep thresholds, or None
        if support is not None and self.cp > 1:
            _, support = self._gather_rollouts(tokens, support)
        tokens, old_logp = self._gather_rollouts(tokens, old_logp)
        ev[1].record()
        if rewards_fn is None:
            gen = torch.Generator(device=self.dev).manual_seed(c.seed + step_index)
            # drawn for the whole job, then cut: a sequence's reward does not depend on the layout
            rewards = torch.bernoulli(torch.full((c.num_seqs,), 0.5, device=self.dev), generator=gen)
            rewards = rewards[self.ctx.dp_rank * B:(self.ctx.dp_rank + 1) * B]
        else:
            rewards = rewards_fn(tokens).float()
        adv = nv.group_advantages(rewards.contiguous(), self.rep_prompts, c.group_size, 1e-6)
        _, ridx = self.engine.response_index(c.seq_len, c.prompt_len)   # response columns of this rank
        Rl = ridx.numel()
        mask = torch.ones(B, Rl, dtype=torch.uint8, device=self.dev)
        old_local = old_logp if self.cp == 1 else old_logp[:, ridx].contiguous()
        ref_logp = self.score(self.ref_params, tokens, support) if self.ref_params is not None else None
        ev[2].record()
        total_active = float(c.num_seqs * R)          # the loss is normalised over the whole job
        self.policy.grad.zero_()
        train_logp = torch.empty(B, Rl, dtype=torch.float32, device=self.dev)
        loss_terms = []
        tmb = c.train_micro_batch_seqs or c.micro_batch_seqs
        for b0 in range(0, B, tmb):
            b1 = min(B, b0 + tmb)

            def dlogp_fn(lp, b0=b0, b1=b1):
                r = nv.grpo_loss(lp.contiguous(), old_local[b0:b1].contiguous(),
                                 ref_logp[b0:b1].contiguous() if ref_logp is not None else None,
                                 adv[b0:b1].contiguous(), mask[b0:b1].contiguous(), clip_lo=c.clip_eps,
                                 clip_hi=c.clip_eps, beta=c.kl_coef, inv_norm=1.0 / total_active,
                                 want_tokens=False)
                loss_terms.append(r["totals"])
                return r["dlogp"]

            lp = self.engine.train_forward_backward(tokens[b0:b1], c.prompt_len, dlogp_fn,
                                                    temperature=c.temperature,
                                                    store_activations=c.store_activations,
                                                    min_keep=None if support is None else support[b0:b1])
            train_logp[b0:b1].copy_(lp)
        tot = torch.stack(loss_terms).sum(0)
        if self.cp > 1:
            # weights are replicated over CP: sum the gradients of the token shards (fixed tree)
            self.ctx.cp_collective.all_reduce_(self.policy.grad)
            pad = torch.zeros(B, R, dtype=torch.float32, device=self.dev)
            pad[:, :Rl] = train_logp
            idx = torch.full((R,), -1, dtype=torch.int64, device=self.dev)
            idx[:Rl] = ridx
            gp, gi = self.ctx.cp_collective.all_gather(pad), self.ctx.cp_collective.all_gather(idx)
            train_logp = torch.empty(B, R, dtype=torch.float32, device=self.dev)
            for r in range(self.cp):                      # every response column has exactly one owner
                m = gi[r] >= 0
                train_logp[:, gi[r][m]] = gp[r][:, m]
            tot = self.ctx.cp_collective.all_gather(tot.contiguous()).sum(0)
        if self.dp > 1:
            # replicas saw different sequences: sum their gradients in the collective's fixed tree
            self.ctx.dp_collective.all_reduce_(self.policy.grad)
            tot = self.ctx.dp_collective.all_gather(tot.contiguous()).sum(0)
        ev[3].record()
        self.opt.step()
        ev[4].record()
        self.phase_events = ev     # rollout, reference scoring, train fwd/bwd, optimizer
        return {"tokens": tokens, "old_logp": old_logp, "train_logp": train_logp, "rewards": rewards,
                "support": support, "loss_sums": tot, "grad_norm": self.opt.last_grad_norm, "total_active": total_active}

    def phase_ms(self) -> dict[str, float]:
        """Device time of the last step's phases (call after a synchronize)."""
        e = self.phase_events
        names = ("rollout", "ref_score", "train_fwd_bwd", "optimizer")
        return {n: e[i].elapsed_time(e[i + 1]) for i, n in enumerate(names)}

    @staticmethod
    def mismatch_count(train_logp: torch.Tensor, rollout_logp: torch.Tensor) -> int:
        return bit_mismatch_count(train_logp, rollout_logp)
