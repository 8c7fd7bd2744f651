"""Typed Python entry points for every ``rlk_*`` function of librlk_b200.so.

Each wrapper validates dtypes / contiguity that the C side cannot see, passes raw device
pointers and the current CUDA stream, and raises on a non-zero return code.  No wrapper falls
back to PyTorch: on a machine with a GPU a missing library is an error.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_uint, c_ulonglong, c_void_p

import torch

from rl_kernel_b200.backends import extension as ext

_ll = c_longlong
LAUNCH_COUNT = 0  # number of native kernel-launching calls made by this process


def _lib():
    return ext.load()


def _count(n: int = 1) -> None:
    global LAUNCH_COUNT
    LAUNCH_COUNT += n


def set_pdl(on: bool) -> bool:
    """Programmatic dependent launch for the library's kernel chains (on by default; the environment
    variable RLK_PDL=0 turns it off at load).  Returns the previous setting."""
    return bool(_lib().rlk_set_pdl(c_int(int(on))))


def det_gemm_swiglu(x: torch.Tensor, wgu: torch.Tensor, act: torch.Tensor, blk: int) -> None:
    """act[M, I] = SwiGLU(x @ wgu^T) for the packed gate/up weight (blocks of ``blk`` rows); the
    gate/up tensor is not materialised.  Same bits as det_gemm + swiglu_fwd."""
    _bf16(x, "x"); _bf16(wgu, "wgu"); _rowmajor2d(act, "act")
    M, K = x.shape
    I = wgu.shape[0] // 2
    rc = _lib().rlk_det_gemm_swiglu(ext.ptr(x), ext.ptr(wgu), ext.ptr(act), c_int(M), c_int(I), c_int(K),
                                    _ll(x.stride(0)), _ll(wgu.stride(0)), _ll(act.stride(0)), c_int(blk),
                                    ext.stream_ptr(x.device))
    ext.check(rc, "det_gemm_swiglu")
    _count()


class static_weights:
    """Context: the B operands (weights) of the GEMMs launched inside were complete before the
    kernel preceding each GEMM was launched, so the kernels may start streaming them while that
    kernel still runs.  Never wrap a GEMM whose B is produced by the kernel right before it."""

    def __enter__(self):
        self._old = _lib().rlk_set_static_b(c_int(1))
        return self

    def __exit__(self, *exc):
        _lib().rlk_set_static_b(c_int(self._old))
        return False


def _bf16(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dtype != torch.bfloat16 or not t.is_cuda:
        raise TypeError(f"{name} must be a CUDA bf16 tensor, got {t.dtype} on {t.device}")
    return t


def _f32(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous():
        raise TypeError(f"{name} must be a contiguous CUDA fp32 tensor, got {t.dtype} on {t.device}")
    return t


def _rowmajor2d(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be 2-D with unit inner stride, got shape {tuple(t.shape)} "
                         f"stride {t.stride()}")
    return t


# ------------------------------------------------------------------------------------- GEMM
def det_gemm_split_leaves(a: torch.Tensor, b: torch.Tensor, scratch: torch.Tensor, *, nchunks: int,
                          tile_n: int = 64) -> int:
    """The chunked few-row GEMM without its tree pass: ``scratch`` [nchunks, M, N] receives one bf16
    partial result per canonical K chunk; returns the element stride between chunks.  The consumer
    (``rmsnorm_fwd_leaves``) evaluates the tree while it loads."""
    _bf16(a, "a"); _bf16(b, "b"); _bf16(scratch, "scratch")
    M, K = a.shape
    N = b.shape[0]
    if scratch.numel() < nchunks * M * N:
        raise ValueError("det_gemm_split_leaves: scratch too small")
    rc = _lib().rlk_det_gemm_split(ext.ptr(a), ext.ptr(b), c_void_p(0), ext.ptr(scratch), c_int(M), c_int(N),
                                   c_int(K), _ll(a.stride(0)), _ll(b.stride(0)), _ll(N), c_int(nchunks),
                                   c_int(tile_n), ext.stream_ptr(a.device))
    ext.check(rc, "det_gemm_split_leaves")
    _count()
    return M * N


def det_gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, *, M: int, N: int, K: int,
             a_mn: bool = False, b_mn: bool = False, nchunks: int = 1, tile_n: int = 0,
             accumulate: bool = False) -> torch.Tensor:
    """out[M,N] (+)= A[M,K] @ B[N,K]^T; see csrc/gemm/det_gemm_sm100.cu for the contract."""
    _bf16(a, "a"); _bf16(b, "b")
    _rowmajor2d(a, "a"); _rowmajor2d(b, "b"); _rowmajor2d(out, "out")
    out_fp32 = 1 if out.dtype == torch.float32 else 0
    if not out_fp32:
        _bf16(out, "out")
    rc = _lib().rlk_det_gemm(ext.ptr(a), ext.ptr(b), ext.ptr(out), c_int(M), c_int(N), c_int(K),
                             _ll(a.stride(0)), _ll(b.stride(0)), _ll(out.stride(0)),
                             c_int(int(a_mn)), c_int(int(b_mn)), c_int(nchunks), c_int(tile_n),
                             c_int(out_fp32), c_int(int(accumulate)), ext.stream_ptr(a.device))
    ext.check(rc, "det_gemm")
    _count()
    return out


def det_gemm_split(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor, *,
                   nchunks: int, tile_n: int = 64) -> torch.Tensor:
    """Chunked GEMM for few rows: one set of CTAs per canonical K chunk + a tree kernel.
    Bitwise equal to ``det_gemm(..., nchunks=nchunks)``. ``scratch``: bf16, >= nchunks*M*ldc elements."""
    _bf16(a, "a"); _bf16(b, "b"); _bf16(out, "out"); _bf16(scratch, "scratch")
    _rowmajor2d(a, "a"); _rowmajor2d(b, "b"); _rowmajor2d(out, "out")
    M, K = a.shape
    N = b.shape[0]
    if scratch.numel() < nchunks * M * out.stride(0):
        raise ValueError("det_gemm_split: scratch too small")
    rc = _lib().rlk_det_gemm_split(ext.ptr(a), ext.ptr(b), ext.ptr(out), ext.ptr(scratch), c_int(M),
                                   c_int(N), c_int(K), _ll(a.stride(0)), _ll(b.stride(0)),
                                   _ll(out.stride(0)), c_int(nchunks), c_int(tile_n),
                                   ext.stream_ptr(a.device))
    ext.check(rc, "det_gemm_split")
    _count(2)
    return out


def lmhead_logp_stats(h: torch.Tensor, w: torch.Tensor, targets: torch.Tensor | None,
                      stats: torch.Tensor, tgt_logit: torch.Tensor, *, vocab_start: int,
                      inv_temp: float, logits_out: torch.Tensor | None = None,
                      min_keep: torch.Tensor | None = None) -> None:
    """``min_keep`` fp32 [M]: restricted sampling support (scaled logits below it count as -inf)."""
    _bf16(h, "h"); _bf16(w, "w"); _rowmajor2d(h, "h"); _rowmajor2d(w, "w")
    M, K = h.shape
    N = w.shape[0]
    assert stats.dtype == torch.float32 and stats.dim() == 3 and stats.shape[2] == 2 and stats.is_contiguous()
    _keep(min_keep, M)
    rc = _lib().rlk_lmhead_logp_stats_keep(ext.ptr(h), ext.ptr(w), c_int(M), c_int(N), c_int(K),
                                           _ll(h.stride(0)), _ll(w.stride(0)), ext.ptr(targets),
                                           _ll(vocab_start), c_float(inv_temp), ext.ptr(min_keep), ext.ptr(stats),
                                           _ll(stats.shape[1]), ext.ptr(tgt_logit), ext.ptr(logits_out),
                                           _ll(logits_out.stride(0) if logits_out is not None else 0),
                                           ext.stream_ptr(h.device))
    ext.check(rc, "lmhead_logp_stats")
    _count()


def _keep(min_keep, rows: int) -> None:
    if min_keep is not None and (min_keep.dtype != torch.float32 or min_keep.numel() != rows or not min_keep.is_contiguous()
                                 or not min_keep.is_cuda):
        raise ValueError(f"min_keep must be a contiguous CUDA fp32 tensor with one value per row ({rows})")


def lmhead_logp_stats_vp(h: torch.Tensor, w: torch.Tensor, targets: torch.Tensor, stats_bufs, tgt_bufs, rank: int,
                         *, vocab_start: int, inv_temp: float, min_keep: torch.Tensor | None = None) -> None:
    """Vocab-parallel fused LM head: this shard's per-tile statistics (and the target logit, if this
    shard owns the target) are stored into every rank's buffers from the GEMM epilogue.
    ``stats_bufs[r]`` [M, ntile, 2] fp32 and ``tgt_bufs[r]`` [M] fp32 are rank r's buffers mapped here."""
    _bf16(h, "h"); _bf16(w, "w"); _rowmajor2d(h, "h"); _rowmajor2d(w, "w")
    M, K = h.shape
    world = len(stats_bufs)
    sp = (c_void_p * world)(*[t.data_ptr() for t in stats_bufs])
    tp = (c_void_p * world)(*[t.data_ptr() for t in tgt_bufs])
    _keep(min_keep, M)
    rc = _lib().rlk_lmhead_logp_stats_vp_keep(ext.ptr(h), ext.ptr(w), c_int(M), c_int(w.shape[0]), c_int(K),
                                              _ll(h.stride(0)), _ll(w.stride(0)), ext.ptr(targets), _ll(vocab_start),
                                              c_float(inv_temp), ext.ptr(min_keep), sp, _ll(stats_bufs[0].shape[1]), tp,
                                              c_int(world), c_int(rank), ext.stream_ptr(h.device))
    ext.check(rc, "lmhead_logp_stats_vp")
    _count()


# ------------------------------------------------------------------------------------- attention
def attn_fwd(q2d: torch.Tensor, k_list: list[torch.Tensor], v_list: list[torch.Tensor],
             o2d: torch.Tensor, lse: torch.Tensor | None, tiles: torch.Tensor, scale: float, *,
             cp_blocks_per_chunk: int = 0, cp_zigzag: bool = False, decode: bool = False,
             page_table: torch.Tensor | None = None, stage: tuple | None = None,
             resume: tuple | None = None) -> None:
    """q2d/o2d: [rows, Hq*128]; k/v: [rows, Hkv*128] (one tensor per source rank).  ``page_table``
    int32: tiles whose last column is > 0 read KV block b from page ``table[col - 1 + b]``.
    ``resume`` = (tile_ext int32 [tiles, 4], state fp32, rows per sequence in a tile, rows between
    sequences in q2d, sequences per tile or 0): rows whose block loop is cut in two launches
    (see ``AttnFwdParams::tile_ext``)."""
    _bf16(q2d, "q"); _rowmajor2d(q2d, "q"); _rowmajor2d(o2d, "o")
    n_src = len(k_list)
    k0 = k_list[0]
    _rowmajor2d(k0, "k")
    kp = (c_void_p * n_src)(*[t.data_ptr() for t in k_list])
    vp = (c_void_p * n_src)(*[t.data_ptr() for t in v_list])
    assert tiles.dtype == torch.int32 and tiles.is_contiguous() and tiles.shape[1] == 12
    rc = _lib().rlk_attn_fwd(ext.ptr(q2d), _ll(q2d.shape[0]), _ll(q2d.shape[1]), _ll(q2d.stride(0)),
                             kp, vp, c_int(n_src), _ll(k0.shape[0]), _ll(k0.shape[1]),
                             _ll(k0.stride(0)), ext.ptr(o2d), _ll(o2d.stride(0)), ext.ptr(lse),
                             ext.ptr(tiles), c_int(tiles.shape[0]), c_float(scale),
                             c_int(cp_blocks_per_chunk), c_int(int(cp_zigzag)), c_int(int(decode)),
                             ext.ptr(page_table), *_stage_args(stage), *_resume_args(resume, tiles),
                             ext.stream_ptr(q2d.device))
    ext.check(rc, "attn_fwd")
    _count()


def _resume_args(resume, tiles):
    if resume is None:
        return c_void_p(0), c_void_p(0), c_int(0), c_int(0), c_int(0)
    ext_t, state, rps, seq_rows, group = resume
    assert ext_t.dtype == torch.int32 and ext_t.is_contiguous() and ext_t.shape == (tiles.shape[0], 4)
    assert state.dtype == torch.float32 and state.is_contiguous()
    return ext.ptr(ext_t), ext.ptr(state), c_int(int(rps)), c_int(int(seq_rows)), c_int(int(group))


def _stage_args(stage):
    """``stage`` = (buffer a, buffer b, int32 flags, rows per rank, this rank) for context-parallel
    staging of remote blocks, or None."""
    if stage is None:
        return c_void_p(0), c_void_p(0), c_void_p(0), c_int(0), c_int(0)
    a, b, flags, rows, rank = stage
    return ext.ptr(a), ext.ptr(b), ext.ptr(flags), c_int(int(rows)), c_int(int(rank))


def attn_bwd_delta(o2d: torch.Tensor, do2d: torch.Tensor, delta: torch.Tensor, T: int, Hq: int) -> None:
    rc = _lib().rlk_attn_bwd_delta(ext.ptr(o2d), _ll(o2d.stride(0)), ext.ptr(do2d),
                                   _ll(do2d.stride(0)), ext.ptr(delta), c_int(T), c_int(Hq),
                                   ext.stream_ptr(o2d.device))
    ext.check(rc, "attn_bwd_delta")
    _count()


def _as_list(x):
    return list(x) if isinstance(x, (list, tuple)) else [x]


def attn_bwd_dq(q2d, do2d, k2d, v2d, lse, delta, dq2d, tiles, scale: float, *,
                cp_blocks_per_chunk: int = 0, cp_zigzag: bool = False, stage: tuple | None = None) -> None:
    """``k2d`` / ``v2d``: one tensor, or one per context-parallel rank (peers' buffers mapped here)."""
    ks, vs = _as_list(k2d), _as_list(v2d)
    n_src, k0 = len(ks), ks[0]
    kp = (c_void_p * n_src)(*[t.data_ptr() for t in ks])
    vp = (c_void_p * n_src)(*[t.data_ptr() for t in vs])
    rc = _lib().rlk_attn_bwd_dq(ext.ptr(q2d), ext.ptr(do2d), _ll(q2d.shape[0]), _ll(q2d.shape[1]),
                                _ll(q2d.stride(0)), _ll(do2d.stride(0)), kp, vp, c_int(n_src),
                                _ll(k0.shape[0]), _ll(k0.shape[1]), _ll(k0.stride(0)),
                                ext.ptr(lse), ext.ptr(delta), ext.ptr(dq2d), _ll(dq2d.stride(0)),
                                ext.ptr(tiles), c_int(tiles.shape[0]), c_float(scale),
                                c_int(cp_blocks_per_chunk), c_int(int(cp_zigzag)), *_stage_args(stage),
                                ext.stream_ptr(dq2d.device))
    ext.check(rc, "attn_bwd_dq")
    _count()


def attn_bwd_dkv(q2d, do2d, k2d, v2d, lse, delta, dk2d, dv2d, kv_tiles, scale: float, *,
                 cp_blocks_per_chunk: int = 0, cp_zigzag: bool = False, stage: tuple | None = None) -> None:
    """``q2d`` / ``do2d`` / ``lse`` / ``delta``: one tensor each, or one per context-parallel rank."""
    qs, dos, ls, ds = _as_list(q2d), _as_list(do2d), _as_list(lse), _as_list(delta)
    n_src, q0, do0 = len(qs), qs[0], dos[0]
    assert len(dos) == len(ls) == len(ds) == n_src
    qp = (c_void_p * n_src)(*[t.data_ptr() for t in qs])
    dop = (c_void_p * n_src)(*[t.data_ptr() for t in dos])
    lp = (c_void_p * n_src)(*[t.data_ptr() for t in ls])
    dp = (c_void_p * n_src)(*[t.data_ptr() for t in ds])
    rc = _lib().rlk_attn_bwd_dkv(qp, dop, c_int(n_src), _ll(q0.shape[0]), _ll(q0.shape[1]),
                                 _ll(q0.stride(0)), _ll(do0.stride(0)), ext.ptr(k2d), ext.ptr(v2d),
                                 _ll(k2d.shape[0]), _ll(k2d.shape[1]), _ll(k2d.stride(0)), lp, dp,
                                 ext.ptr(dk2d), ext.ptr(dv2d), _ll(dk2d.stride(0)), ext.ptr(kv_tiles),
                                 c_int(kv_tiles.shape[0]), c_float(scale), c_int(cp_blocks_per_chunk),
                                 c_int(int(cp_zigzag)), *_stage_args(stage), ext.stream_ptr(dk2d.device))
    ext.check(rc, "attn_bwd_dkv")
    _count()


# ------------------------------------------------------------------------------------- norm / rope
def rmsnorm_fwd(x, w, y, eps: float, *, res=None, res_out=None, rstd_out=None) -> None:
    rows, H = x.shape
    rc = _lib().rlk_rmsnorm_fwd(ext.ptr(x), ext.ptr(res), ext.ptr(w), ext.ptr(y), ext.ptr(res_out),
                                ext.ptr(rstd_out), c_int(rows), c_int(H), c_float(eps),
                                ext.stream_ptr(x.device))
    ext.check(rc, "rmsnorm_fwd")
    _count()


def rmsnorm_fwd_leaves(leaves, chunk_stride: int, nchunks: int, res, w, y, res_out, eps: float) -> None:
    """y = rmsnorm(tree(leaves) + res) * w; res_out = tree(leaves) + res (see det_gemm_split_leaves)."""
    rows, H = y.shape
    rc = _lib().rlk_rmsnorm_fwd_leaves(ext.ptr(leaves), _ll(chunk_stride), c_int(nchunks), ext.ptr(res), ext.ptr(w),
                                       ext.ptr(y), ext.ptr(res_out), c_int(rows), c_int(H), c_float(eps),
                                       ext.stream_ptr(y.device))
    ext.check(rc, "rmsnorm_fwd_leaves")
    _count()


def rmsnorm_bwd_scratch_elems(rows: int, H: int) -> int:
    fn = _lib().rlk_rmsnorm_bwd_scratch_elems
    fn.restype = c_longlong
    return int(fn(c_int(rows), c_int(H)))


def rmsnorm_bwd(x, w, dy, dx, scratch, eps: float, *, dres=None, dw_bf16=None, dw_f32=None,
                accumulate_dw: bool = False) -> None:
    rows, H = x.shape
    rc = _lib().rlk_rmsnorm_bwd(ext.ptr(x), ext.ptr(w), ext.ptr(dy), ext.ptr(dres), ext.ptr(dx),
                                ext.ptr(scratch), ext.ptr(dw_bf16), ext.ptr(dw_f32),
                                c_int(int(accumulate_dw)), c_int(rows), c_int(H), c_float(eps),
                                ext.stream_ptr(x.device))
    ext.check(rc, "rmsnorm_bwd")
    _count(2)


def qk_norm_rope_fwd(qkv, q_w, k_w, cos_tab, sin_tab, pos, q_out, k_out, v_out, *, Hq: int, Hkv: int,
                     eps: float, kv_slot=None) -> None:
    T = qkv.shape[0]
    assert pos.dtype == torch.int32 and cos_tab.dtype == torch.float32
    rc = _lib().rlk_qk_norm_rope_fwd(ext.ptr(qkv), _ll(qkv.stride(0)), ext.ptr(q_w), ext.ptr(k_w),
                                     ext.ptr(cos_tab), ext.ptr(sin_tab), ext.ptr(pos), ext.ptr(kv_slot),
                                     ext.ptr(q_out), _ll(q_out.stride(0)), ext.ptr(k_out),
                                     ext.ptr(v_out), _ll(k_out.stride(0)), c_int(T), c_int(Hq),
                                     c_int(Hkv), c_float(eps), c_void_p(0), c_void_p(0),
                                     ext.stream_ptr(qkv.device))
    ext.check(rc, "qk_norm_rope_fwd")
    _count()


def qk_norm_rope_bwd_scratch_elems(T: int) -> int:
    fn = _lib().rlk_qk_norm_rope_bwd_scratch_elems
    fn.restype = c_longlong
    return int(fn(c_int(T)))


def qk_norm_rope_bwd(qkv, q_w, k_w, cos_tab, sin_tab, pos, dq, dk, dv, dqkv, scratch, dqw, dkw, *,
                     Hq: int, Hkv: int, eps: float, accumulate_dw: bool) -> None:
    T = qkv.shape[0]
    rc = _lib().rlk_qk_norm_rope_bwd(ext.ptr(qkv), _ll(qkv.stride(0)), ext.ptr(q_w), ext.ptr(k_w),
                                     ext.ptr(cos_tab), ext.ptr(sin_tab), ext.ptr(pos), ext.ptr(dq),
                                     _ll(dq.stride(0)), ext.ptr(dk), ext.ptr(dv), _ll(dk.stride(0)),
                                     ext.ptr(dqkv), _ll(dqkv.stride(0)), ext.ptr(scratch),
                                     ext.ptr(dqw), ext.ptr(dkw), c_int(int(accumulate_dw)), c_int(T),
                                     c_int(Hq), c_int(Hkv), c_float(eps), ext.stream_ptr(qkv.device))
    ext.check(rc, "qk_norm_rope_bwd")
    _count(4)


def qk_norm_rope_bwd_canonical(qkv, q_w, k_w, cos_tab, sin_tab, pos, dq, dk, dv, dqkv, scratch, dqk, *,
                               Hq: int, Hkv: int, eps: float, accumulate_dw: bool) -> None:
    """Backward of the fused QK-norm + RoPE with canonical gain gradients: ``dqk`` [256] bf16 =
    [d q_norm | d k_norm], one bf16 leaf per KV group combined by a balanced tree, so that the bits
    do not depend on how many of the groups this rank holds (the tensor-parallel all-reduce
    continues the same tree)."""
    T = qkv.shape[0]
    rc = _lib().rlk_qk_norm_rope_bwd_canonical(ext.ptr(qkv), _ll(qkv.stride(0)), ext.ptr(q_w), ext.ptr(k_w),
                                               ext.ptr(cos_tab), ext.ptr(sin_tab), ext.ptr(pos), ext.ptr(dq),
                                               _ll(dq.stride(0)), ext.ptr(dk), ext.ptr(dv), _ll(dk.stride(0)),
                                               ext.ptr(dqkv), _ll(dqkv.stride(0)), ext.ptr(scratch), ext.ptr(dqk),
                                               c_int(int(accumulate_dw)), c_int(T), c_int(Hq), c_int(Hkv),
                                               c_float(eps), ext.stream_ptr(qkv.device))
    ext.check(rc, "qk_norm_rope_bwd_canonical")
    _count(2)


# ------------------------------------------------------------------------------------- activation
def swiglu_fwd(gu, out, I: int, blk: int | None = None, rows_limit=None) -> None:
    """``rows_limit``: int32 device scalar; rows at or beyond it are skipped."""
    rc = _lib().rlk_swiglu_fwd_dyn(ext.ptr(gu), _ll(gu.stride(0)), ext.ptr(out), _ll(out.stride(0)),
                                   c_int(gu.shape[0]), c_int(I), c_int(blk or I), ext.ptr(rows_limit),
                                   ext.stream_ptr(gu.device))
    ext.check(rc, "swiglu_fwd")
    _count()


def swiglu_bwd(gu, dout, dgu, I: int, blk: int | None = None, rows_limit=None) -> None:
    rc = _lib().rlk_swiglu_bwd_dyn(ext.ptr(gu), _ll(gu.stride(0)), ext.ptr(dout), _ll(dout.stride(0)),
                                   ext.ptr(dgu), _ll(dgu.stride(0)), c_int(gu.shape[0]), c_int(I),
                                   c_int(blk or I), ext.ptr(rows_limit), ext.stream_ptr(gu.device))
    ext.check(rc, "swiglu_bwd")
    _count()


def swiglu_split_fwd(gate, up, out) -> None:
    """out [rows, I] = silu(gate) * up for gate / up / out in separate 2-D bf16 tensors (unit inner stride,
    row strides multiples of 8 elements, 16-byte aligned)."""
    rc = _lib().rlk_swiglu_split_fwd(ext.ptr(gate), _ll(gate.stride(0)), ext.ptr(up), _ll(up.stride(0)), ext.ptr(out),
                                     _ll(out.stride(0)), c_int(gate.shape[0]), c_int(gate.shape[1]),
                                     ext.stream_ptr(gate.device))
    ext.check(rc, "swiglu_split_fwd")
    _count()


def swiglu_split_bwd(gate, up, dout, dgate, dup) -> None:
    rc = _lib().rlk_swiglu_split_bwd(ext.ptr(gate), _ll(gate.stride(0)), ext.ptr(up), _ll(up.stride(0)), ext.ptr(dout),
                                     _ll(dout.stride(0)), ext.ptr(dgate), _ll(dgate.stride(0)), ext.ptr(dup),
                                     _ll(dup.stride(0)), c_int(gate.shape[0]), c_int(gate.shape[1]),
                                     ext.stream_ptr(gate.device))
    ext.check(rc, "swiglu_split_bwd")
    _count()


# ------------------------------------------------------------------------------------- embedding
def embedding_fwd(ids, w, out, vocab_start: int = 0) -> None:
    assert ids.dtype == torch.int64
    rc = _lib().rlk_embedding_fwd(ext.ptr(ids), ext.ptr(w), ext.ptr(out), c_int(ids.numel()),
                                  c_int(w.shape[1]), _ll(vocab_start), _ll(w.shape[0]),
                                  ext.stream_ptr(w.device))
    ext.check(rc, "embedding_fwd")
    _count()


def embedding_bwd(sorted_ids, order, dy, dw, vocab_start: int = 0) -> None:
    rc = _lib().rlk_embedding_bwd(ext.ptr(sorted_ids), ext.ptr(order), ext.ptr(dy), ext.ptr(dw),
                                  c_int(sorted_ids.numel()), c_int(dw.shape[1]), _ll(vocab_start),
                                  _ll(dw.shape[0]), ext.stream_ptr(dw.device))
    ext.check(rc, "embedding_bwd")
    _count()


# ------------------------------------------------------------------------------------- logp
def logits_tile_stats(logits, targets, stats, tgt_logit, *, vocab_start: int, inv_temp: float,
                      row_indices=None, min_keep=None) -> None:
    """``row_indices`` int64 [rows]: output row r scores logits row ``row_indices[r]``.
    ``min_keep`` fp32 [rows]: scaled logits below the row's value are outside the support."""
    n_local = logits.shape[1]
    rows = logits.shape[0] if row_indices is None else row_indices.numel()
    _keep(min_keep, rows)
    rc = _lib().rlk_logits_tile_stats_keep(ext.ptr(logits), _ll(logits.stride(0)), ext.ptr(targets),
                                           ext.ptr(stats), _ll(stats.shape[1]), ext.ptr(tgt_logit),
                                           c_int(rows), c_int(n_local), _ll(vocab_start), c_float(inv_temp),
                                           ext.ptr(row_indices), ext.ptr(min_keep), ext.stream_ptr(logits.device))
    ext.check(rc, "logits_tile_stats")
    _count()


def logp_merge(stats, tgt_logit, logp, lse) -> None:
    rows, n_tiles = stats.shape[0], stats.shape[1]
    rc = _lib().rlk_logp_merge(ext.ptr(stats), _ll(n_tiles), c_int(n_tiles), ext.ptr(tgt_logit),
                               ext.ptr(logp), ext.ptr(lse), c_int(rows), ext.stream_ptr(stats.device))
    ext.check(rc, "logp_merge")
    _count()


def replay_tile_stats(logits, targets, replay_ids, stats_compact, tgt_logit, *, vocab_start: int, inv_temp: float,
                      row_indices=None) -> None:
    """Restricted-support statistics from id lists: ``replay_ids`` int64 [rows, K<=64] (global ids),
    ``stats_compact`` fp32 [rows, K, 2] (touched tiles in ascending order, then (-inf, 0) fillers)."""
    _bf16(logits, "logits"); _rowmajor2d(logits, "logits")
    rows, K = replay_ids.shape
    if replay_ids.dtype != torch.int64 or not replay_ids.is_contiguous() or not 0 < K <= 64:
        raise ValueError("replay_ids must be contiguous int64 [rows, K] with K <= 64")
    if stats_compact.dtype != torch.float32 or tuple(stats_compact.shape) != (rows, K, 2) or not stats_compact.is_contiguous():
        raise ValueError("stats_compact must be contiguous fp32 [rows, K, 2]")
    rc = _lib().rlk_replay_tile_stats(ext.ptr(logits), _ll(logits.stride(0)), ext.ptr(targets), ext.ptr(replay_ids),
                                      c_int(K), ext.ptr(stats_compact), ext.ptr(tgt_logit), c_int(rows),
                                      c_int(logits.shape[1]), _ll(vocab_start), c_float(inv_temp), ext.ptr(row_indices),
                                      ext.stream_ptr(logits.device))
    ext.check(rc, "replay_tile_stats")
    _count()


def dlogits_(logits, targets, lse, g, *, vocab_start: int, inv_temp: float, g_lse=None, min_keep=None) -> None:
    rows, n_local = logits.shape
    _keep(min_keep, rows)
    rc = _lib().rlk_dlogits_keep(ext.ptr(logits), _ll(logits.stride(0)), ext.ptr(targets), ext.ptr(lse),
                                 ext.ptr(g), ext.ptr(g_lse), ext.ptr(min_keep), c_int(rows), c_int(n_local),
                                 _ll(vocab_start), c_float(inv_temp), ext.stream_ptr(logits.device))
    ext.check(rc, "dlogits")
    _count()


# ------------------------------------------------------------------------------------- loss
def grpo_loss(logp, old_logp, ref_logp, adv, mask_u8, *, clip_lo: float, clip_hi: float, beta: float,
              inv_norm: float, want_tokens: bool = True):
    B, L = logp.shape
    dev = logp.device
    dlogp = torch.empty_like(logp)
    loss_tok = torch.empty_like(logp) if want_tokens else None
    kl_tok = torch.empty_like(logp) if want_tokens else None
    ratio_tok = torch.empty_like(logp) if want_tokens else None
    seq_sums = torch.empty(B, 4, device=dev, dtype=torch.float32)
    totals = torch.empty(8, device=dev, dtype=torch.float32)
    rc = _lib().rlk_grpo_loss(ext.ptr(logp), ext.ptr(old_logp), ext.ptr(ref_logp), ext.ptr(adv),
                              ext.ptr(mask_u8), ext.ptr(loss_tok), ext.ptr(kl_tok), ext.ptr(ratio_tok),
                              ext.ptr(dlogp), ext.ptr(seq_sums), ext.ptr(totals), c_int(B), c_int(L),
                              c_float(clip_lo), c_float(clip_hi), c_float(beta), c_float(inv_norm),
                              ext.stream_ptr(dev))
    ext.check(rc, "grpo_loss")
    _count(2)
    return dict(dlogp=dlogp, loss_tok=loss_tok, kl_tok=kl_tok, ratio_tok=ratio_tok,
                seq_sums=seq_sums, totals=totals)


def group_advantages(rewards, groups: int, n: int, eps: float):
    adv = torch.empty_like(rewards)
    rc = _lib().rlk_group_advantages(ext.ptr(rewards), ext.ptr(adv), c_int(groups), c_int(n),
                                     c_float(eps), ext.stream_ptr(rewards.device))
    ext.check(rc, "group_advantages")
    _count()
    return adv


# ------------------------------------------------------------------------------------- sampling
_SAMPLE_SCRATCH: dict[tuple, torch.Tensor] = {}


def _sample_scratch(rows: int, device) -> torch.Tensor:
    key = (rows, str(device))
    t = _SAMPLE_SCRATCH.get(key)
    if t is None:
        t = torch.empty(rows * 8 * 12 // 8 + 8, dtype=torch.int64, device=device)
        _SAMPLE_SCRATCH[key] = t
    return t


def sample_gumbel(logits, out_ids, out_val, *, vocab_start: int, inv_temp: float, seed: int, step: int,
                  greedy: bool = False, min_keep=None, row_keys=None) -> None:
    rows, n_local = logits.shape
    scratch = _sample_scratch(rows, logits.device)
    rc = _lib().rlk_sample_gumbel(ext.ptr(logits), _ll(logits.stride(0)), ext.ptr(min_keep),
                                  ext.ptr(row_keys), ext.ptr(out_ids), ext.ptr(out_val),
                                  ext.ptr(scratch), c_int(rows),
                                  c_int(n_local), _ll(vocab_start), c_float(inv_temp),
                                  c_ulonglong(seed), c_uint(step), c_int(int(greedy)),
                                  ext.stream_ptr(logits.device))
    ext.check(rc, "sample_gumbel")
    _count(2)


# ------------------------------------------------------------------------------------- optimizer
def sample_keep_threshold(logits, out_thr, *, inv_temp: float, top_k: int = 0, top_p: float = 1.0) -> None:
    """out_thr[row] = smallest scaled logit kept under top-k / top-p (no sort; csrc/sampling/sampling.cu)."""
    _bf16(logits, "logits"); _rowmajor2d(logits, "logits")
    rc = _lib().rlk_sample_keep_threshold(ext.ptr(logits), _ll(logits.stride(0)), c_int(logits.shape[0]),
                                          c_int(logits.shape[1]), c_float(inv_temp), c_int(int(top_k)),
                                          c_float(float(top_p)), ext.ptr(out_thr), ext.stream_ptr(logits.device))
    ext.check(rc, "sample_keep_threshold")
    _count()


def adamw(master, m, v, grad, param, *, lr: float, beta1: float, beta2: float, eps: float,
          weight_decay: float, step: int, grad_scale=None) -> None:
    rc = _lib().rlk_adamw(ext.ptr(master), ext.ptr(m), ext.ptr(v), ext.ptr(grad), ext.ptr(param),
                          _ll(master.numel()), c_float(lr), c_float(beta1), c_float(beta2),
                          c_float(eps), c_float(weight_decay), c_int(step), ext.ptr(grad_scale),
                          ext.stream_ptr(master.device))
    ext.check(rc, "adamw")
    _count()


def sumsq_bins(grad, bins) -> None:
    assert bins.dtype == torch.int64 and bins.numel() == 256
    rc = _lib().rlk_sumsq_bins(ext.ptr(grad), _ll(grad.numel()), ext.ptr(bins), ext.stream_ptr(grad.device))
    ext.check(rc, "sumsq_bins")
    _count()


# ------------------------------------------------------------------------------------- MoE
def _ptr_array(tensors):
    ts = _as_list(tensors)
    return (c_void_p * len(ts))(*[t.data_ptr() for t in ts]), len(ts)


def grouped_gemm(a, b, c, tiles, n_tiles, *, a_mn: bool = False, b_mn: bool = False,
                 accumulate: bool = False) -> None:
    """Tile-list driven expert GEMM (csrc/moe/grouped_gemm_sm100.cu).  ``tiles`` int32 [max, 8] and
    ``n_tiles`` int32 [1] live on the device and come from ``moe_tiles``."""
    _bf16(a, "a"); _bf16(b, "b"); _bf16(c, "c")
    _rowmajor2d(a, "a"); _rowmajor2d(b, "b"); _rowmajor2d(c, "c")
    rc = _lib().rlk_grouped_gemm(ext.ptr(a), _ll(a.shape[0]), _ll(a.shape[1]), _ll(a.stride(0)),
                                 ext.ptr(b), _ll(b.shape[0]), _ll(b.shape[1]), _ll(b.stride(0)),
                                 ext.ptr(c), _ll(c.stride(0)), ext.ptr(tiles), ext.ptr(n_tiles),
                                 c_int(tiles.shape[0]), c_int(int(a_mn)), c_int(int(b_mn)),
                                 c_int(int(accumulate)), ext.stream_ptr(a.device))
    ext.check(rc, "grouped_gemm")
    _count()


def moe_router_topk(logits, idx, w, probs=None, counts=None) -> None:
    """logits fp32 [T, E] -> idx int32 [T, K] (ascending expert ids), w fp32 [T, K]."""
    T, E = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous() and idx.dtype == torch.int32
    rc = _lib().rlk_moe_router_topk(ext.ptr(logits), c_int(T), c_int(E), c_int(idx.shape[1]), ext.ptr(idx),
                                    ext.ptr(w), ext.ptr(probs), ext.ptr(counts), ext.stream_ptr(logits.device))
    ext.check(rc, "moe_router_topk")
    _count()


def moe_router_bwd(idx, w, dw, dlogits) -> None:
    T, K = idx.shape
    rc = _lib().rlk_moe_router_bwd(ext.ptr(idx), ext.ptr(w), ext.ptr(dw), c_int(T), c_int(K),
                                   c_int(dlogits.shape[1]), ext.ptr(dlogits), ext.stream_ptr(idx.device))
    ext.check(rc, "moe_router_bwd")
    _count()


def moe_plan(counts_all, rank: int, send_row0, loc, rows_used) -> None:
    W, E = counts_all.shape
    rc = _lib().rlk_moe_plan(ext.ptr(counts_all), c_int(W), c_int(rank), c_int(E), ext.ptr(send_row0),
                             ext.ptr(loc), ext.ptr(rows_used), ext.stream_ptr(counts_all.device))
    ext.check(rc, "moe_plan")
    _count()


def moe_tiles(loc, kind: int, n_cols: int, k_dim: int, b_mn: bool, m_out: int, tiles, n_tiles) -> None:
    rc = _lib().rlk_moe_tiles(ext.ptr(loc), c_int(loc.shape[0]), c_int(kind), c_int(n_cols), c_int(k_dim),
                              c_int(int(b_mn)), c_int(m_out), ext.ptr(tiles), ext.ptr(n_tiles),
                              c_int(tiles.shape[0]), ext.stream_ptr(loc.device))
    ext.check(rc, "moe_tiles")
    _count()


def moe_slots(idx, E: int, send_row0, slot_row) -> None:
    rc = _lib().rlk_moe_slots(ext.ptr(idx), c_int(idx.numel()), c_int(E), ext.ptr(send_row0),
                              ext.ptr(slot_row), ext.stream_ptr(idx.device))
    ext.check(rc, "moe_slots")
    _count()


def moe_dispatch(x, scale, idx, slot_row, E_loc: int, dst_bufs) -> None:
    """Row t of ``x`` goes to row slot_row[t, k] of ``dst_bufs[owner of idx[t, k]]`` for every k."""
    pa, n = _ptr_array(dst_bufs)
    d0 = _as_list(dst_bufs)[0]
    rc = _lib().rlk_moe_dispatch(ext.ptr(x), _ll(x.stride(0)), ext.ptr(scale), ext.ptr(idx), ext.ptr(slot_row),
                                 c_int(idx.numel()), c_int(idx.shape[1]), c_int(E_loc), c_int(x.shape[1]), pa,
                                 c_int(n), _ll(d0.stride(0)), ext.stream_ptr(x.device))
    ext.check(rc, "moe_dispatch")
    _count()


def moe_combine(base, w, idx, slot_row, E_loc: int, src_bufs, out) -> None:
    pa, n = _ptr_array(src_bufs)
    s0 = _as_list(src_bufs)[0]
    rc = _lib().rlk_moe_combine(ext.ptr(base), _ll(base.stride(0) if base is not None else 0), ext.ptr(w),
                                ext.ptr(idx), ext.ptr(slot_row), c_int(idx.shape[0]), c_int(idx.shape[1]),
                                c_int(E_loc), c_int(out.shape[1]), pa, c_int(n), _ll(s0.stride(0)), ext.ptr(out),
                                _ll(out.stride(0)), ext.stream_ptr(out.device))
    ext.check(rc, "moe_combine")
    _count()


def moe_combine_dw(dout, idx, slot_row, E_loc: int, src_bufs, dw) -> None:
    pa, n = _ptr_array(src_bufs)
    s0 = _as_list(src_bufs)[0]
    rc = _lib().rlk_moe_combine_dw(ext.ptr(dout), _ll(dout.stride(0)), ext.ptr(idx), ext.ptr(slot_row),
                                   c_int(idx.numel()), c_int(idx.shape[1]), c_int(E_loc), c_int(dout.shape[1]),
                                   pa, c_int(n), _ll(s0.stride(0)), ext.ptr(dw), ext.stream_ptr(dout.device))
    ext.check(rc, "moe_combine_dw")
    _count()


def moe_zero_pad(loc, buf) -> None:
    rc = _lib().rlk_moe_zero_pad(ext.ptr(loc), c_int(loc.shape[0]), ext.ptr(buf), _ll(buf.stride(0)),
                                 c_int(buf.shape[1]), ext.stream_ptr(buf.device))
    ext.check(rc, "moe_zero_pad")
    _count()


def sumsq_bins_f32(grad, bins) -> None:
    """Exact fp32 sum of squares: ``bins`` int64 [768] (three 16-bit limbs per exponent)."""
    assert grad.dtype == torch.float32 and bins.dtype == torch.int64 and bins.numel() == 768
    rc = _lib().rlk_sumsq_bins_f32(ext.ptr(grad), _ll(grad.numel()), ext.ptr(bins), ext.stream_ptr(grad.device))
    ext.check(rc, "sumsq_bins_f32")
    _count()


def rope(x: torch.Tensor, pos: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, out: torch.Tensor, *, heads: int,
         head_dim: int, inverse: bool = False) -> torch.Tensor:
    """NeoX RoPE of x [rows, heads*head_dim] (bf16 or fp32, row stride free) at ``pos`` [rows] int32 from
    the fp32 tables cos/sin [max_pos, head_dim/2]; ``inverse`` rotates back (the backward).  ``out`` may
    be ``x``."""
    if x.dtype not in (torch.bfloat16, torch.float32) or out.dtype != x.dtype:
        raise TypeError("rope: x and out must both be bf16 or both fp32")
    if pos.dtype != torch.int32 or not pos.is_contiguous():
        raise TypeError("rope: pos must be contiguous int32")
    _f32(cos, "cos"); _f32(sin, "sin")
    if x.dim() != 2 or out.shape != x.shape or x.stride(1) != 1 or out.stride(1) != 1:
        raise ValueError("rope: x/out must be 2-D with unit inner stride")
    rc = _lib().rlk_rope(ext.ptr(x), _ll(x.stride(0)), ext.ptr(pos), ext.ptr(cos), ext.ptr(sin), ext.ptr(out),
                         _ll(out.stride(0)), _ll(x.shape[0]), c_int(heads), c_int(head_dim), c_int(cos.shape[0]),
                         c_int(int(inverse)), c_int(0 if x.dtype == torch.bfloat16 else 1), ext.stream_ptr(x.device))
    ext.check(rc, "rope")
    _count()
    return out
