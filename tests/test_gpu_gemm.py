"""det_gemm on a B200: accuracy against fp32, and the bitwise invariances of its contract."""
import pytest
import torch

from tests.gpu_util import dev, sync_and_check

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _mk(M, N, K, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn(M, K, device=dev(), generator=g).to(BF)
    b = torch.randn(N, K, device=dev(), generator=g).to(BF)
    return a, b


def _gemm(a, b, M, N, K, **kw):
    from rl_kernel_b200.backends import native as nv

    out = torch.empty(M, N, device=dev(), dtype=kw.pop("dtype", BF))
    nv.det_gemm(a, b, out, M=M, N=N, K=K, **kw)
    sync_and_check()
    return out


@pytest.mark.parametrize("shape", [(128, 256, 64), (200, 512, 1024), (1024, 4096, 4096)])
def test_accuracy_and_tile_invariance(shape):
    M, N, K = shape
    a, b = _mk(M, N, K)
    ref = a.float() @ b.float().t()
    outs = {bn: _gemm(a, b, M, N, K, tile_n=bn) for bn in (256, 192, 128, 64, 32)}
    tol = 2 ** -8 * ref.abs().max().item() + 1e-3
    assert (outs[256].float() - ref).abs().max().item() <= tol
    for bn in (192, 128, 64, 32):
        assert torch.equal(outs[256], outs[bn]), f"tile_n={bn} changed bits"
    f32 = _gemm(a, b, M, N, K, tile_n=128, dtype=torch.float32)
    assert torch.equal(f32.to(BF), outs[128])


def test_decode_shape_picks_a_one_wave_tile_and_keeps_the_bits():
    # 64 rows against the gate/up projection: the kernel's own choice (192-wide tiles, one wave)
    # must give the bits of every other tile width
    M, N, K = 64, 24576, 1024
    a, b = _mk(M, N, K)
    assert torch.equal(_gemm(a, b, M, N, K), _gemm(a, b, M, N, K, tile_n=128))


@pytest.mark.parametrize("M", [8, 64, 128])
def test_fused_gate_up_swiglu_equals_gemm_then_swiglu(M):
    from rl_kernel_b200.backends import native as nv

    I, K, blk = 1536, 512, 192          # gate / up rows interleaved in blocks of 192
    a = (torch.randn(M, K, device=dev()) * 0.5).to(BF)
    wgu = (torch.randn(2 * I, K, device=dev()) * 0.05).to(BF)
    gu = torch.empty(M, 2 * I, device=dev(), dtype=BF)
    nv.det_gemm(a, wgu, gu, M=M, N=2 * I, K=K)
    ref = torch.empty(M, I, device=dev(), dtype=BF)
    nv.swiglu_fwd(gu, ref, I, blk)
    act = torch.zeros(M, I, device=dev(), dtype=BF)
    nv.det_gemm_swiglu(a, wgu, act, blk)
    sync_and_check()
    assert torch.equal(act, ref)


def test_batch_invariance():
    M, N, K = 777, 1024, 2048
    a, b = _mk(M, N, K, 1)
    full = _gemm(a, b, M, N, K)
    for rows in (1, 5, 64, 130):
        part = _gemm(a[:rows].contiguous(), b, rows, N, K)
        assert torch.equal(part, full[:rows])


def test_operand_majors_agree():
    M, N, K = 256, 512, 1024
    a, b = _mk(M, N, K, 2)
    base = _gemm(a, b, M, N, K)
    at, bt = a.t().contiguous(), b.t().contiguous()
    assert torch.equal(_gemm(a, bt, M, N, K, b_mn=True), base)
    assert torch.equal(_gemm(at, bt, M, N, K, a_mn=True, b_mn=True), base)
    assert torch.equal(_gemm(at, b, M, N, K, a_mn=True), base)


@pytest.mark.parametrize("nchunks", [2, 4, 8])
def test_canonical_chunk_tree(nchunks):
    from rl_kernel_b200.backends import native as nv

    M, N, K = 200, 512, 1024
    a, b = _mk(M, N, K, 3)
    got = _gemm(a, b, M, N, K, nchunks=nchunks)
    kc = K // nchunks
    leaves = [_gemm(a[:, i * kc:(i + 1) * kc], b[:, i * kc:(i + 1) * kc], M, N, kc, tile_n=128) for i in range(nchunks)]
    while len(leaves) > 1:
        leaves = [(leaves[i].float() + leaves[i + 1].float()).to(BF) for i in range(0, len(leaves), 2)]
    assert torch.equal(got, leaves[0])
    # 128x256 tiles with the tree stack in the L2-resident scratch give the same bits
    assert torch.equal(_gemm(a, b, M, N, K, nchunks=nchunks, tile_n=256), got)
    bt = b.t().contiguous()
    assert torch.equal(_gemm(a, bt, M, N, K, nchunks=nchunks, tile_n=256, b_mn=True), got)
    # the split (small-M) form gives the same bits
    out = torch.empty(M, N, device=dev(), dtype=BF)
    scratch = torch.empty(nchunks * M * N, device=dev(), dtype=BF)
    for tn in (32, 64, 128):
        nv.det_gemm_split(a, b, out, scratch, nchunks=nchunks, tile_n=tn)
        sync_and_check()
        assert torch.equal(out, got)


def test_accumulate():
    M, N, K = 128, 256, 512
    a, b = _mk(M, N, K, 4)
    from rl_kernel_b200.backends import native as nv

    c0 = torch.randn(M, N, device=dev()).to(BF)
    c = c0.clone()
    nv.det_gemm(a, b, c, M=M, N=N, K=K, accumulate=True)
    sync_and_check()
    ref = c0.float() + a.float() @ b.float().t()
    assert (c.float() - ref).abs().max().item() <= 2 ** -7 * ref.abs().max().item()


def test_bad_shapes_are_rejected():
    from rl_kernel_b200.backends import native as nv
    from rl_kernel_b200.backends.extension import NativeLibraryError

    a, b = _mk(16, 24, 64)
    with pytest.raises(NativeLibraryError):
        nv.det_gemm(a, b[:, :60].contiguous(), torch.empty(16, 24, device=dev(), dtype=BF), M=16, N=24, K=60)
    with pytest.raises(NativeLibraryError):
        nv.det_gemm(a, b, torch.empty(16, 24, device=dev(), dtype=BF), M=16, N=24, K=64, nchunks=3)
