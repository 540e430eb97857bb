"""tcgen05 GEMM kernels against fp32 PyTorch references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _C():
    from deepep_ascend_b200 import _native
    return _native.load()


@pytest.mark.parametrize('M,N,K', [(128, 128, 64), (128, 128, 256), (256, 384, 512), (1000, 520, 1096), (4096, 2048, 7168),
                                   (1024, 896, 1024), (2048, 7168, 512)])
def test_bf16_gemm(M, N, K):
    """Shapes that take each of the three tile widths (128, 224 and 256 columns; the launcher picks by tile count)."""
    C = _C()
    g = torch.Generator(device='cuda').manual_seed(M + N)
    a = torch.randn(M, K, device='cuda', generator=g).bfloat16()
    b = torch.randn(N, K, device='cuda', generator=g).bfloat16()
    c = C.gemm_nt(a, b)
    torch.cuda.synchronize()
    assert C.gemm_error(0) == 0
    ref = a.float() @ b.float().t()
    err = (c.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-2, err


def _quant_b(b):
    """[G, N, K] -> e4m3 with one fp32 scale per 128 x 128 block."""
    G, N, K = b.shape
    nb, kb = (N + 127) // 128, (K + 127) // 128
    bp = torch.zeros(G, nb * 128, kb * 128, device=b.device)
    bp[:, :N, :K] = b
    blocks = bp.view(G, nb, 128, kb, 128)
    amax = blocks.abs().amax(dim=(2, 4)).clamp(1e-4)
    q = (blocks * (448.0 / amax)[:, :, None, :, None]).to(torch.float8_e4m3fn).view(G, nb * 128, kb * 128)[:, :N, :K].contiguous()
    return q, (amax / 448.0).contiguous()


@pytest.mark.parametrize('M,N,K,G', [(128, 128, 128, 1), (256, 256, 512, 1), (512, 384, 1024, 4), (1024, 2048, 7168, 8)])
def test_fp8_blockscaled_grouped_gemm(M, N, K, G):
    from deepep_ascend_b200.utils.math import per_token_cast_back
    C = _C()
    g = torch.Generator(device='cuda').manual_seed(K + G)
    a = torch.randn(M, K, device='cuda', generator=g).bfloat16()
    b = torch.randn(G, N, K, device='cuda', generator=g) * 0.1
    qa, sfa = C.per_token_cast_to_fp8(a, False, False)
    qb, sfb = _quant_b(b)
    tiles = (M + 127) // 128
    tile_group = (torch.arange(tiles, device='cuda', dtype=torch.int32) % G).contiguous()
    if tiles > 2:
        tile_group[1] = -1
    c = torch.full((M, N), 7.0, device='cuda', dtype=torch.bfloat16)
    C.gemm_nt(qa, qb, sfa, sfb, tile_group, c)
    torch.cuda.synchronize()
    assert C.gemm_error(0) == 0
    a_deq = per_token_cast_back(qa, sfa).float()
    kb = (K + 127) // 128
    for t in range(tiles):
        rows = slice(t * 128, min(M, (t + 1) * 128))
        grp = int(tile_group[t])
        if grp < 0:
            assert bool((c[rows] == 7.0).all())
            continue
        b_deq = qb[grp].float().view(N, -1) * sfb[grp].repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)[:, :K]
        ref = a_deq[rows] @ b_deq.t()
        err = (c[rows].float() - ref).abs().max().item()
        assert err <= 2e-2 * ref.abs().max().item() + 1e-2, (t, err)


@pytest.mark.parametrize('M,N,segs', [(128, 128, [64, 0, 192]), (384, 520, [128, 256, 0, 0, 640]), (2048, 7168, [1152, 1024, 0, 1280])])
def test_k_grouped_gemm(M, N, segs):
    """out[e] = a_t[:, seg_e] @ b_t[:, seg_e]^T (weight gradients of a grouped layer); empty segments give zeros."""
    from deepep_ascend_b200.ops import gemm as G
    C = _C()
    g = torch.Generator(device='cuda').manual_seed(M + N)
    K = sum(segs)
    a_t = torch.randn(M, K, device='cuda', generator=g).bfloat16()
    b_t = torch.randn(N, K, device='cuda', generator=g).bfloat16()
    off = torch.tensor([0] + list(torch.tensor(segs).cumsum(0)), dtype=torch.int32, device='cuda')
    out = G.gemm_kgrouped(a_t, b_t, off)
    torch.cuda.synchronize()
    assert C.gemm_error(0) == 0
    assert out.shape == (len(segs), M, N)
    k0 = 0
    for e, n in enumerate(segs):
        ref = a_t[:, k0:k0 + n].float() @ b_t[:, k0:k0 + n].float().t()
        err = (out[e].float() - ref).abs().max().item()
        assert err <= 2e-2 * max(ref.abs().max().item(), 1.0) + 1e-2, (e, err)
        if n == 0:
            assert out[e].abs().max().item() == 0
        k0 += n
