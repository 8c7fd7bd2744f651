"""Pipeline parallelism: stage-to-stage activation / gradient transfers on NCCL point-to-point
(the one hot path that stays on NCCL) overlapped with compute, and a 1F1B schedule over the
engine's stage interface.

The reference pins pipeline parallelism to 1 and only forwards the setting to Megatron / vLLM
(rl_engine/integrations/orchestrators/vime/experiments/dense/run_arm.py:650).  Here a stage is a
``Qwen3Engine`` built over ``PackedParams(layers=(first, end), has_embed=..., has_head=...)``.

Boundary tensors: forward sends the last layer's (block output, residual) pair, [tokens, hidden]
bf16 each -- the next stage's fused add + norm then sees exactly the operands of the single-GPU
run, so log-probs and gradients are bitwise those of the unsplit model; backward sends one
[tokens, hidden] gradient.  Transfers are issued on a side stream from per-micro-batch buffers,
so sending micro-batch i overlaps computing micro-batch i + 1.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def split_layers(num_layers: int, n_stages: int) -> list[tuple[int, int]]:
    """Contiguous layer ranges, earlier stages take the remainder."""
    base, extra = divmod(num_layers, n_stages)
    out, l0 = [], 0
    for s in range(n_stages):
        n = base + (1 if s < extra else 0)
        out.append((l0, l0 + n))
        l0 += n
    return out


def one_f_one_b(stage: int, n_stages: int, n_micro: int) -> list[tuple[str, int]]:
    """The 1F1B order of ('F', i) / ('B', i) steps for one stage: n_stages - stage - 1 warm-up
    forwards, then alternating forward / backward, then the remaining backwards."""
    warm = min(n_stages - stage - 1, n_micro)
    steps = [("F", i) for i in range(warm)]
    f, b = warm, 0
    while b < n_micro:
        if f < n_micro:
            steps.append(("F", f))
            f += 1
        steps.append(("B", b))
        b += 1
    return steps


class StageLink:
    """NCCL send / receive with the neighbouring stages on a dedicated stream."""

    def __init__(self, stage: int, n_stages: int, device: torch.device, *, group=None, ranks: list[int] | None = None):
        self.stage, self.n, self.dev, self.group = stage, n_stages, device, group
        self.ranks = ranks if ranks is not None else list(range(n_stages))   # global rank of every stage
        self.stream = torch.cuda.Stream(device)

    def _run(self, ops):
        """Issue on the side stream after everything already queued on the compute stream; returns
        an event the consumer (or the buffer's next writer) waits for."""
        cur = torch.cuda.current_stream(self.dev)
        self.stream.wait_stream(cur)
        with torch.cuda.stream(self.stream):
            for r in dist.batch_isend_irecv(ops):
                r.wait()
            ev = torch.cuda.Event()
            ev.record(self.stream)
        return ev

    def send(self, tensors: list[torch.Tensor], to_stage: int):
        return self._run([dist.P2POp(dist.isend, t, self.ranks[to_stage], group=self.group) for t in tensors])

    def recv(self, tensors: list[torch.Tensor], from_stage: int):
        ev = self._run([dist.P2POp(dist.irecv, t, self.ranks[from_stage], group=self.group) for t in tensors])
        torch.cuda.current_stream(self.dev).wait_event(ev)


class PipelineTrainer:
    """Runs ``n_micro`` micro-batches through this rank's stage with the 1F1B schedule."""

    def __init__(self, engine, link: StageLink):
        self.eng, self.link = engine, link
        self.stage, self.n = link.stage, link.n
        self.first, self.last = engine.first_stage, engine.last_stage
        self._bufs: dict = {}
        self._send_done: dict = {}

    def _buf(self, name: str, i: int, shape) -> torch.Tensor:
        key = (name, i % (self.n + 1), tuple(shape))
        if key not in self._bufs:
            self._bufs[key] = torch.empty(shape, dtype=torch.bfloat16, device=self.eng.dev)
        ev = self._send_done.pop(key, None)
        if ev is not None:
            torch.cuda.current_stream(self.eng.dev).wait_event(ev)     # an earlier send still reads it
        return self._bufs[key]

    def run(self, micro_tokens: list[torch.Tensor], resp_start: int, dlogp_fn, *, temperature: float = 1.0):
        """``micro_tokens``: the same list of [nseq, S] token tensors on every stage (ids are cheap;
        only the last stage needs them for targets, the first for the embedding).  Returns the list
        of log-prob tensors on the last stage, [] elsewhere."""
        eng, H = self.eng, self.eng.spec.hidden_size
        states: dict[int, object] = {}
        logps = []
        for kind, i in one_f_one_b(self.stage, self.n, len(micro_tokens)):
            tok = micro_tokens[i]
            T = tok.numel()
            if kind == "F":
                stage_in = None
                if not self.first:
                    x, r = self._buf("in_x", i, (T, H)), self._buf("in_r", i, (T, H))
                    self.link.recv([x, r], self.stage - 1)
                    stage_in = (x, r)
                if self.last:
                    # forward + loss + backward of the same micro-batch back to back
                    logps.append(eng.train_forward_backward(tok, resp_start, lambda lp, i=i: dlogp_fn(lp, i),
                                                            temperature=temperature, stage_in=stage_in).clone())
                    if not self.first:
                        g = self._buf("out_g", i, (T, H))
                        g.copy_(eng.stage_input_grad)
                        self._send_done[("out_g", i % (self.n + 1), (T, H))] = self.link.send([g], self.stage - 1)
                else:
                    st, (x_out, r_out) = eng.stage_forward(tok, stage_in, slot=i % self.n)
                    states[i] = st
                    sx, sr = self._buf("out_x", i, (T, H)), self._buf("out_r", i, (T, H))
                    sx.copy_(x_out)
                    sr.copy_(r_out)
                    ev = self.link.send([sx, sr], self.stage + 1)
                    self._send_done[("out_x", i % (self.n + 1), (T, H))] = ev
                    self._send_done[("out_r", i % (self.n + 1), (T, H))] = ev
            elif not self.last:
                gin = self._buf("in_g", i, (T, H))
                self.link.recv([gin], self.stage + 1)
                ds = eng.stage_backward(states.pop(i), tok, gin)
                if not self.first:
                    g = self._buf("out_g", i, (T, H))
                    g.copy_(ds)
                    self._send_done[("out_g", i % (self.n + 1), (T, H))] = self.link.send([g], self.stage - 1)
        return logps
