"""Fused MoE layer (dispatch -> FP8 grouped GEMM -> SwiGLU -> FP8 grouped GEMM -> weighted combine) and its
backward pass on one GPU (a group of one rank), against a plain fp32 PyTorch statement of the layer."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize('T,H,I,E,K', [(200, 256, 128, 4, 2), (512, 1024, 512, 8, 4)])
def test_fused_moe_forward_backward(T, H, I, E, K):
    from deepep_ascend_b200 import ElasticBuffer
    from deepep_ascend_b200.models.moe import FusedMoE, moe_reference
    from deepep_ascend_b200.utils.math import calc_diff
    torch.manual_seed(0)
    buf = ElasticBuffer(None, num_max_tokens_per_rank=T, hidden=H, num_topk=K, enable_expand=True, num_experts=E,
                        expert_alignment=128)
    try:
        layer = FusedMoE(buf, E, H, I, init_std=0.05, num_sms=16)
        x = torch.randn(T, H, device='cuda').bfloat16().requires_grad_(True)
        scores = torch.softmax(torch.randn(T, E, device='cuda'), dim=-1)
        w, idx = scores.topk(K, dim=-1)
        idx[::7, 0] = -1
        w = w.clone().requires_grad_(True)
        out = layer(x, idx, w)
        g = torch.randn_like(out)
        out.backward(g)
        torch.cuda.synchronize()
        buf.check_status()

        xr = x.detach().float().requires_grad_(True)
        wr = w.detach().clone().requires_grad_(True)
        w13 = layer.w13.detach().float().requires_grad_(True)
        w2 = layer.w2.detach().float().requires_grad_(True)
        ref = moe_reference(xr, idx, wr, w13, w2)
        ref.backward(g.float())
        assert calc_diff(out.float(), ref) < 3e-3, calc_diff(out.float(), ref)
        assert calc_diff(x.grad.float(), xr.grad) < 3e-3, calc_diff(x.grad.float(), xr.grad)
        assert calc_diff(w.grad, wr.grad) < 3e-3, calc_diff(w.grad, wr.grad)
        assert calc_diff(layer.w2.grad.float(), w2.grad) < 3e-3, calc_diff(layer.w2.grad.float(), w2.grad)
        assert calc_diff(layer.w13.grad.float(), w13.grad) < 3e-3, calc_diff(layer.w13.grad.float(), w13.grad)
    finally:
        buf.destroy()
